// Launchers for the tensor-parallel fused GEMMs (the kernel lives in gemm/gemm_kernel.cuh):
//
//   st_ag_gemm   Y[T, N_local] = epilogue(gather(X_shard)[T, K] · Wᵀ)   all-gather → GEMM
//   st_gemm_rs   Y_shard[T/W, N] = reduce-scatter(A[T, K_local] · Wᵀ)   GEMM → reduce-scatter
//
// Both take B either K-major ([N, K], forward) or MN-major ([K, N], data gradient).  Peer
// pointers and signal areas come from symmetric allocations made by the Python side
// (spiraltorch_b200/parallel/symm.py).  With world == 1 the launchers degenerate to the
// local case (the "peer" is this GPU), which is how the single-GPU tests exercise them.
//
// The reference has no tensor parallelism; the baseline these are measured against is
// NCCL all-gather / reduce-scatter around the same GEMM kernel.
#include "../gemm/gemm_kernel.cuh"
#include <cstring>

struct StPeerGroup {
  int world, rank;
  unsigned epoch;
  unsigned long long signals[st::kMaxRanks];
  unsigned long long signals_mc;
};
namespace st {
void fill_peer_group(PeerGroup& g, const StPeerGroup& s);
}

namespace {
using namespace st;
using namespace st::gemm;

constexpr int BN = 256;
constexpr int STAGES = 4;

// The all-gather variant runs a 3-stage operand pipeline so that the push ring (and its barriers)
// fits behind the GEMM's shared memory; it has two extra warps.
constexpr int AG_STAGES = 3;
constexpr int AG_EXTRA_SMEM = AG_RING_SLOTS * AG_RING_CHUNK + 64;

template <bool B_MN, int COMM, int ST = STAGES>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const OutMaps& tmC, const CUtensorMap& tmA_local,
           const GemmParams& p, const GemmComm& cm, int grid, cudaStream_t stream) {
  using L = SmemLayout<BN, ST>;
  constexpr int SMEM = L::TOTAL + ((COMM == COMM_AG && ST == AG_STAGES) ? AG_EXTRA_SMEM : 0);
  static_assert(SMEM <= 232448, "dynamic shared memory above the 227 KB limit");
  auto kern = gemm_bf16_kernel<BN, ST, false, B_MN, COMM>;
  static bool configured[st::kMaxDevices] = {false};   // the attribute is per device
  const int dev = st::current_device();
  if (!configured[dev]) {
    ST_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured[dev] = true;
  }
  kern<<<grid, COMM == COMM_AG ? NUM_THREADS_AG : NUM_THREADS, SMEM, stream>>>(tmA, tmB, tmC, tmA_local, p, cm);
  ST_CUDA_CHECK(cudaGetLastError());
  return ST_OK;
}

bool make_maps(CUtensorMap* tmA, CUtensorMap* tmB, const void* A, const void* B, int M, int N, int K,
               long long lda, long long ldb, int b_mn) {
  uint64_t dims[3], strides[2];
  uint32_t box[3];
  dims[0] = K; dims[1] = M; dims[2] = 1; box[0] = BK; box[1] = BM; box[2] = 1;
  strides[0] = (uint64_t)lda * 2; strides[1] = (uint64_t)lda * 2 * M;
  if (!encode_tmap(tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
    return false;
  if (!b_mn) {
    dims[0] = K; dims[1] = N; box[0] = BK; box[1] = BN;
    strides[1] = (uint64_t)ldb * 2 * N;
  } else {
    dims[0] = N; dims[1] = K; box[0] = 64; box[1] = BK;
    strides[1] = (uint64_t)ldb * 2 * K;
  }
  strides[0] = (uint64_t)ldb * 2;
  return encode_tmap(tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

struct StAgGemmArgs {
  StPeerGroup g;
  unsigned long long x_shard;                  // bf16 [T/W, K] contiguous (this rank's rows)
  unsigned long long gather_peers[st::kMaxRanks];  // bf16 [T, K] on every rank (symmetric)
  unsigned long long gather_mc;                // multicast alias of the gather buffer or 0
  unsigned long long B;                        // bf16 weights: [N, K] or, b_mn, [K, N]
  unsigned long long C;                        // bf16 [T, N]
  unsigned long long bias, aux_out, aux_in;    // optional epilogue operands (bf16)
  long long ldb, ldc, ld_aux_out, ld_aux_in;
  int T, N, K;
  int b_mn, act;
  float alpha;
  int sub_per_chunk;   // arrival granularity per rank shard (1, 2, 4, 8 or 16)
  int comm_ctas;       // unused (every CTA pushes a slice of the shard)
  int slot_enter, slot_arrive;   // slot_arrive: counter area of THIS sub_per_chunk value (world * 16 words)
  unsigned arrive_target;  // cumulative arrivals per counter: launches with this sub_per_chunk so far
                           // times st_ag_arrivals_per_launch()
  unsigned long long trace;  // optional device buffer of [3 * grid][4] 64-bit time stamps, or 0
  int stages;                // 0: choose by world size; 3 or 4: force that operand-pipeline depth
  int local_in_place;        // x_shard IS this rank's slot of its own gather buffer: nothing is copied locally
  int max_ctas;              // 0: one CTA per SM; > 0: a smaller grid, which leaves SMs to a concurrent kernel.  Every
                             // rank must pass the same value: the grid is also the arrival count per counter.
};

// Arrivals every (source, sub-chunk) counter receives per launch: one per CTA of the grid.
ST_API int st_ag_arrivals_per_launch() {
  const int sms = st::sm_count();
  return sms > 0 ? sms : 148;
}

// The same for a launch whose grid is limited to `max_ctas` (0 = no limit).
ST_API int st_ag_arrivals_for(int max_ctas) {
  const int full = st_ag_arrivals_per_launch();
  return max_ctas > 0 && max_ctas < full ? max_ctas : full;
}

ST_API int st_ag_gemm(const StAgGemmArgs* a, void* stream_v) {
  if (!a) return st::fail(ST_ERR_INVALID, "ag_gemm: null args");
  const int W = a->g.world;
  if (W < 1 || W > st::kMaxRanks) return st::fail(ST_ERR_INVALID, "ag_gemm: bad world size");
  if (a->T % (W * BM) != 0) return st::fail(ST_ERR_INVALID, "ag_gemm: T must be a multiple of world*128");
  const int rows = a->T / W;
  if (a->sub_per_chunk > kMaxSubChunks) return st::fail(ST_ERR_INVALID, "ag_gemm: at most 16 sub-chunks per shard");
  if (a->sub_per_chunk < 1 || rows % (a->sub_per_chunk * BM) != 0)
    return st::fail(ST_ERR_INVALID, "ag_gemm: shard rows must be a multiple of sub_per_chunk*128");
  if (a->K % 8 || a->ldb % 8) return st::fail(ST_ERR_INVALID, "ag_gemm: K and ldb must be multiples of 8");
  const void* gathered = reinterpret_cast<const void*>(a->gather_peers[a->g.rank]);
  CUtensorMap tmA, tmB;
  if (!make_maps(&tmA, &tmB, gathered, reinterpret_cast<const void*>(a->B), a->T, a->N, a->K, a->K, a->ldb, a->b_mn))
    return ST_ERR_CUDA;
  GemmParams p{};
  p.C = reinterpret_cast<void*>(a->C);
  p.ldc = a->ldc;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a->bias);
  p.aux_out = reinterpret_cast<__nv_bfloat16*>(a->aux_out);
  p.ld_aux_out = a->ld_aux_out;
  p.aux_in = reinterpret_cast<const __nv_bfloat16*>(a->aux_in);
  p.ld_aux_in = a->ld_aux_in;
  p.M = a->T; p.N = a->N; p.K = a->K;
  p.alpha = a->alpha; p.act = a->act;
  p.batch = 1;
  p.err = st::error_word();
  GemmComm cm{};
  st::fill_peer_group(cm.g, a->g);
  cm.rows_per_chunk = rows;
  cm.sub_per_chunk = a->sub_per_chunk;
  cm.slot_enter = a->slot_enter;
  cm.slot_arrive = a->slot_arrive;
  cm.arrive_target = a->arrive_target;
  cm.trace = reinterpret_cast<unsigned long long*>(a->trace);
  cm.sub_major = 0;
  cm.local_in_place = a->local_in_place;
  if (a->local_in_place &&
      a->x_shard != a->gather_peers[a->g.rank] + (unsigned long long)a->g.rank * rows * a->K * 2)
    return st::fail(ST_ERR_INVALID, "ag_gemm: local_in_place needs x_shard to be this rank's slot of the gather buffer");
  cm.src_shard = reinterpret_cast<const __nv_bfloat16*>(a->x_shard);
  for (int i = 0; i < st::kMaxRanks; ++i) cm.gather_peers[i] = reinterpret_cast<__nv_bfloat16*>(a->gather_peers[i]);
  cm.gather_mc = reinterpret_cast<__nv_bfloat16*>(a->gather_mc);
  const int grid = st_ag_arrivals_for(a->max_ctas);   // every CTA pushes, whether or not it has tiles
  cm.gemm_ctas = grid;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  OutMaps tmC;
  memset(&tmC, 0, sizeof(tmC));
  p.use_tma_store = ((a->ldc & 7) == 0 && (a->C & 15) == 0) ? 1 : 0;
  if (p.use_tma_store) {
    uint64_t dims[3] = {(uint64_t)a->N, (uint64_t)a->T, 1};
    uint64_t strides[2] = {(uint64_t)a->ldc * 2, (uint64_t)a->ldc * 2 * a->T};
    uint32_t box[3] = {64, 32, 1};
    if (!encode_tmap(&tmC.m[0], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, reinterpret_cast<const void*>(a->C), dims,
                     strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return ST_ERR_CUDA;
  }
  CUtensorMap tmA_local;
  {
    uint64_t dims[3] = {(uint64_t)a->K, (uint64_t)rows, 1};
    uint64_t strides[2] = {(uint64_t)a->K * 2, (uint64_t)a->K * 2 * rows};
    uint32_t box[3] = {BK, BM, 1};
    if (!encode_tmap(&tmA_local, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, reinterpret_cast<const void*>(a->x_shard),
                     dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return ST_ERR_CUDA;
  }
  // communication-bound (many ranks, thin per-rank GEMM): deeper push ring, 3 operand stages;
  // compute-bound: full 4-stage operand pipeline, small ring
  const bool comm_bound = a->stages == 3 || (a->stages == 0 && W >= 6);
  if (comm_bound) {
    if (a->b_mn) return launch<true, COMM_AG, AG_STAGES>(tmA, tmB, tmC, tmA_local, p, cm, grid, stream);
    return launch<false, COMM_AG, AG_STAGES>(tmA, tmB, tmC, tmA_local, p, cm, grid, stream);
  }
  if (a->b_mn) return launch<true, COMM_AG, 4>(tmA, tmB, tmC, tmA_local, p, cm, grid, stream);
  return launch<false, COMM_AG, 4>(tmA, tmB, tmC, tmA_local, p, cm, grid, stream);
}

struct StGemmRsArgs {
  StPeerGroup g;
  unsigned long long A;                          // bf16 [T, K_local]
  unsigned long long B;                          // bf16 [N, K_local] or, b_mn, [K_local, N]
  unsigned long long stage_peers[st::kMaxRanks]; // bf16 [W][T/W, N] staging on every rank (symmetric)
  unsigned long long out;                        // bf16 [T/W, N] reduced shard (local)
  unsigned long long residual;                   // optional bf16 [T/W, N] added in the reduction
  long long lda, ldb;
  int T, N, K;
  int b_mn;
  float alpha;
  int slot_enter, slot_done;
  unsigned done_target;                          // cumulative warp arrivals expected per row block
  unsigned long long stage_mc;                   // unused
  unsigned long long trace;                      // optional [grid][4] 64-bit time stamps, or 0
  int groups;                                    // row-block groups per chunk for the remote / local interleave;
                                                 // 0 = choose (up to 8), 1 = all remote tiles first, local last
  int lag;                                       // groups by which a local group trails its remote group (0 = 1)
  int max_ctas;                                  // 0: one CTA per SM; > 0: a smaller grid (SMs left to a concurrent kernel)
};

ST_API int st_gemm_rs(const StGemmRsArgs* a, void* stream_v) {
  if (!a) return st::fail(ST_ERR_INVALID, "gemm_rs: null args");
  const int W = a->g.world;
  if (W < 1 || W > st::kMaxRanks) return st::fail(ST_ERR_INVALID, "gemm_rs: bad world size");
  if (a->T % (W * BM) != 0) return st::fail(ST_ERR_INVALID, "gemm_rs: T must be a multiple of world*128");
  if (a->N % 8 || a->K % 8 || a->lda % 8 || a->ldb % 8)
    return st::fail(ST_ERR_INVALID, "gemm_rs: N, K, lda, ldb must be multiples of 8");
  CUtensorMap tmA, tmB;
  if (!make_maps(&tmA, &tmB, reinterpret_cast<const void*>(a->A), reinterpret_cast<const void*>(a->B), a->T,
                 a->N, a->K, a->lda, a->ldb, a->b_mn))
    return ST_ERR_CUDA;
  GemmParams p{};
  p.C = nullptr;  // the epilogue addresses the owners' staging areas
  p.ldc = a->N;
  p.M = a->T; p.N = a->N; p.K = a->K;
  p.alpha = a->alpha;
  p.batch = 1;
  p.err = st::error_word();
  GemmComm cm{};
  st::fill_peer_group(cm.g, a->g);
  cm.rows_per_chunk = a->T / W;
  cm.sub_per_chunk = 1;
  cm.slot_enter = a->slot_enter;
  cm.slot_done = a->slot_done;
  cm.done_target = a->done_target;
  for (int i = 0; i < st::kMaxRanks; ++i) cm.stage_peers[i] = reinterpret_cast<__nv_bfloat16*>(a->stage_peers[i]);
  {
    const int tiles_m_chunk = a->T / W / BM;
    int G = a->groups;
    if (G <= 0) {
      // a group should hold at least one full wave of remote tiles, or the interleave only adds waiting
      G = 8;
      const int tiles_n = (a->N + BN - 1) / BN;
      while (G > 1 && (tiles_m_chunk % G != 0 || (long long)(W - 1) * (tiles_m_chunk / G) * tiles_n < st::sm_count())) G >>= 1;
    }
    if (G < 1 || tiles_m_chunk % G != 0) return st::fail(ST_ERR_INVALID, "gemm_rs: groups must divide the row blocks per rank");
    cm.rs_groups = W == 1 ? 1 : G;
    cm.rs_lag = a->lag > 0 ? a->lag : 1;
  }
  cm.rs_out = reinterpret_cast<__nv_bfloat16*>(a->out);
  cm.rs_residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
  const int tiles = (a->T / BM) * ((a->N + BN - 1) / BN);
  int grid = st::sm_count();
  if (a->max_ctas > 0 && grid > a->max_ctas) grid = a->max_ctas;
  if (grid > tiles) grid = tiles;
  cm.gemm_ctas = grid;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  OutMaps tmC;
  memset(&tmC, 0, sizeof(tmC));
  p.use_tma_store = 1;
  const int rows = a->T / W;
  cm.trace = reinterpret_cast<unsigned long long*>(a->trace);
  for (int q = 0; q < W; ++q) {
    // this rank's slot inside owner q's staging area; for the rows this rank owns, the output itself
    const char* base = q == a->g.rank ? reinterpret_cast<const char*>(a->out)
                                      : reinterpret_cast<const char*>(a->stage_peers[q]) + (size_t)a->g.rank * rows * a->N * 2;
    uint64_t dims[3] = {(uint64_t)a->N, (uint64_t)rows, 1};
    uint64_t strides[2] = {(uint64_t)a->N * 2, (uint64_t)a->N * 2 * rows};
    uint32_t box[3] = {64, 32, 1};
    if (!encode_tmap(&tmC.m[q], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B))
      return ST_ERR_CUDA;
  }
  if (a->b_mn) return launch<true, COMM_RS>(tmA, tmB, tmC, tmA, p, cm, grid, stream);
  return launch<false, COMM_RS>(tmA, tmB, tmC, tmA, p, cm, grid, stream);
}

// Number of warp arrivals one launch of st_gemm_rs adds to every row-block counter: four epilogue
// warps per tile of every OTHER rank (the owner does not count its own tiles).
ST_API int st_gemm_rs_arrivals_per_launch(int world, int N) { return (world - 1) * ((N + BN - 1) / BN) * 4; }
