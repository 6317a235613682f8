// C entry points for callers that can only pass plain buffers and receive C strings (the COBOL bridge of the
// reference: bindings/cobol_bridge/src/lib.rs:14-104): a resonator handle, a description of a coefficient vector as a
// resonance narrative, and the matching free functions.
//
// The coefficient vector is taken as all five resonance channels at once (homotopy flow, functor linearisation,
// recursive objective, infinity projection, infinity energy), as the reference bridge does, and the summary sentence is
// the one the text resonator gives for such a resonance (crates/st-text/src/lib.rs:656-720): dominant band, its
// share, total energy and the observed curvature -sqrt(homotopy energy).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#define ST_HOST_API extern "C" __attribute__((visibility("default")))

namespace {
struct ResonanceHandle {
  float curvature;
  float temperature;
};

constexpr float kEpsilon = 1.1920929e-07f;
const char* const kBandLabels[5] = {"Above band accelerating curvature", "Here band weaving functor linearisation",
                                    "Beneath band anchoring recursive objective", "\xE2\x88\x9E projection tightening geodesics",
                                    "\xE2\x88\x9E hierarchy storing latent energy"};
}  // namespace

// A non-negative curvature is mirrored to a negative one of at least 1e-3 in magnitude, a non-positive temperature to a
// positive one likewise; null on allocation failure.
ST_HOST_API void* st_cobol_new_resonator(float curvature, float temperature) {
  if (!(curvature < 0.0f)) curvature = -std::fmax(std::fabs(curvature), 1.0e-3f);
  if (!(temperature > 0.0f)) temperature = std::fmax(std::fabs(temperature), 1.0e-3f);
  if (!std::isfinite(curvature) || !std::isfinite(temperature)) return nullptr;
  auto* h = new (std::nothrow) ResonanceHandle{curvature, temperature};
  return h;
}

ST_HOST_API void st_cobol_free_resonator(void* handle) { delete static_cast<ResonanceHandle*>(handle); }

// 0 on success (*out_summary receives a heap string for st_cobol_free_string), -1 for null / negative arguments, -2 for an
// empty or non-finite coefficient vector, -3 when the summary cannot be allocated.
ST_HOST_API int st_cobol_describe(void* handle, const float* values, int len, char** out_summary) {
  if (!handle || !values || !out_summary || len < 0) return -1;
  if (len == 0) return -2;
  double energy = 0.0;
  for (int i = 0; i < len; ++i) {
    if (!std::isfinite(values[i])) return -2;
    energy += static_cast<double>(values[i]) * values[i];
  }
  const float band = static_cast<float>(energy);          // every channel carries the same coefficients
  const float total = 5.0f * band;
  char buf[256];
  if (total <= kEpsilon) {
    std::snprintf(buf, sizeof(buf), "Resonance geometry is quiescent; no meaningful curvature pulses detected.");
  } else {
    const float share = std::fmin(std::fmax(band / total, 0.0f), 1.0f);
    const float curvature = band > 0.0f ? -std::sqrt(band) : -1.0f;
    // equal energies keep their channel order, so the first band is the dominant one
    std::snprintf(buf, sizeof(buf), "%s commanding %.1f%% of the field while total energy sits at %.3f with curvature %+.3f.", kBandLabels[0],
                  share * 100.0f, total, curvature);
  }
  const size_t n = std::strlen(buf) + 1;
  char* out = static_cast<char*>(std::malloc(n));
  if (!out) return -3;
  std::memcpy(out, buf, n);
  *out_summary = out;
  return 0;
}

ST_HOST_API void st_cobol_free_string(char* ptr) { std::free(ptr); }
