"""
    SpiralTorch

Julia wrapper over the tensor-level C ABI of `libst_host` (`include/spiraltorch_b200.h`): host tensors, a worker
runtime, the basic algebra with fused epilogues and the roundtable band classifier.  Names follow the Julia binding of
the reference (bindings/julia/src/SpiralTorch.jl: `Tensor`, `Runtime`, `matmul`, `roundtable_classify`, `to_array`, ...).

The library is found through `ENV["SPIRALTORCH_LIB"]`, else `spiraltorch_b200/_native/libst_host.so` relative to this
file, else the loader's search path.  Matrices cross the boundary row-major; Julia's column-major arrays are
transposed on the way in and out, so `to_array(Tensor(A)) == Float32.(A)`.
"""
module SpiralTorch

using Libdl

export Tensor, Runtime, RoundtableSummary, version, shape, elements, to_array, add, sub, hadamard, matmul, matmul_bias_relu,
       matmul_bias_gelu, scale, transpose_tensor, reshape_tensor, row_softmax, random_uniform, random_normal, worker_count,
       roundtable_classify, last_error, clear_error!

const _lib = Ref{Ptr{Cvoid}}(C_NULL)

function _candidate_paths()
    paths = String[]
    haskey(ENV, "SPIRALTORCH_LIB") && push!(paths, ENV["SPIRALTORCH_LIB"])
    push!(paths, normpath(joinpath(@__DIR__, "..", "..", "..", "spiraltorch_b200", "_native", "libst_host.so")))
    push!(paths, "libst_host")
    return paths
end

function load_library!()
    _lib[] != C_NULL && return _lib[]
    for path in _candidate_paths()
        handle = Libdl.dlopen(path; throw_error=false)
        if handle !== nothing
            _lib[] = handle
            return handle
        end
    end
    error("libst_host not found; set ENV[\"SPIRALTORCH_LIB\"] (tried: $(join(_candidate_paths(), ", ")))")
end

_sym(name::Symbol) = Libdl.dlsym(load_library!(), name)

function last_error()
    n = ccall(_sym(:spiraltorch_last_error_length), Csize_t, ())
    n == 0 && return ""
    buf = Vector{UInt8}(undef, n + 1)
    ccall(_sym(:spiraltorch_last_error_message), Csize_t, (Ptr{UInt8}, Csize_t), buf, length(buf))
    return String(buf[1:n])
end

clear_error!() = ccall(_sym(:spiraltorch_clear_last_error), Cvoid, ())

function _fail(context::AbstractString)
    msg = last_error()
    clear_error!()
    error(isempty(msg) ? "$context failed" : "$context: $msg")
end

version() = unsafe_string(ccall(_sym(:spiraltorch_version), Cstring, ()))

# ---- tensors ---------------------------------------------------------------------------------------------------
mutable struct Tensor
    handle::Ptr{Cvoid}
end

function _wrap_tensor(handle::Ptr{Cvoid}, context::AbstractString)
    handle == C_NULL && _fail(context)
    t = Tensor(handle)
    finalizer(close, t)
    return t
end

function Base.close(t::Tensor)
    if t.handle != C_NULL
        ccall(_sym(:spiraltorch_tensor_free), Cvoid, (Ptr{Cvoid},), t.handle)
        t.handle = C_NULL
    end
    return nothing
end

_handle(t::Tensor, context) = t.handle == C_NULL ? error("$context: tensor is closed") : t.handle

Tensor(rows::Integer, cols::Integer) =
    _wrap_tensor(ccall(_sym(:spiraltorch_tensor_zeros), Ptr{Cvoid}, (Csize_t, Csize_t), rows, cols), "tensor_zeros")
Tensor(dims::Tuple{Integer,Integer}) = Tensor(dims[1], dims[2])

function Tensor(data::AbstractMatrix{<:Real})
    rows, cols = size(data)
    dense = Float32.(permutedims(data))                      # row-major order for the library
    GC.@preserve dense _wrap_tensor(ccall(_sym(:spiraltorch_tensor_from_dense), Ptr{Cvoid}, (Csize_t, Csize_t, Ptr{Cfloat}, Csize_t),
                                          rows, cols, dense, length(dense)), "tensor_from_dense")
end
Tensor(data::AbstractVector{<:Real}) = Tensor(reshape(data, 1, :))
function Tensor(data::AbstractVector{<:Real}, dims::Tuple{Integer,Integer})
    length(data) == dims[1] * dims[2] || error("tensor_from_dense: data length does not match rows * cols")
    dense = Float32.(collect(data))                          # already row-major
    GC.@preserve dense _wrap_tensor(ccall(_sym(:spiraltorch_tensor_from_dense), Ptr{Cvoid}, (Csize_t, Csize_t, Ptr{Cfloat}, Csize_t),
                                          dims[1], dims[2], dense, length(dense)), "tensor_from_dense")
end

function shape(t::Tensor)
    r, c = Ref{Csize_t}(0), Ref{Csize_t}(0)
    ok = ccall(_sym(:spiraltorch_tensor_shape), Bool, (Ptr{Cvoid}, Ref{Csize_t}, Ref{Csize_t}), _handle(t, "tensor_shape"), r, c)
    ok || _fail("tensor_shape")
    return (Int(r[]), Int(c[]))
end

elements(t::Tensor) = Int(ccall(_sym(:spiraltorch_tensor_elements), Csize_t, (Ptr{Cvoid},), _handle(t, "tensor_elements")))

function to_array(t::Tensor)
    rows, cols = shape(t)
    flat = Vector{Float32}(undef, rows * cols)
    if !isempty(flat)
        ok = ccall(_sym(:spiraltorch_tensor_copy_data), Bool, (Ptr{Cvoid}, Ptr{Cfloat}, Csize_t), t.handle, flat, length(flat))
        ok || _fail("tensor_copy_data")
    end
    return permutedims(reshape(flat, cols, rows))
end

Base.copyto!(dest::AbstractMatrix{<:Real}, t::Tensor) = copyto!(dest, to_array(t))
Base.size(t::Tensor) = shape(t)

function _seed(seed)
    seed === nothing ? (UInt64(0), false) : (UInt64(seed), true)
end

function random_uniform(rows::Integer, cols::Integer, min::Real, max::Real; seed::Union{Nothing,Integer}=nothing)
    s, has = _seed(seed)
    _wrap_tensor(ccall(_sym(:spiraltorch_tensor_random_uniform), Ptr{Cvoid}, (Csize_t, Csize_t, Cfloat, Cfloat, UInt64, Bool),
                       rows, cols, min, max, s, has), "tensor_random_uniform")
end

function random_normal(rows::Integer, cols::Integer, mean::Real, std::Real; seed::Union{Nothing,Integer}=nothing)
    s, has = _seed(seed)
    _wrap_tensor(ccall(_sym(:spiraltorch_tensor_random_normal), Ptr{Cvoid}, (Csize_t, Csize_t, Cfloat, Cfloat, UInt64, Bool),
                       rows, cols, mean, std, s, has), "tensor_random_normal")
end

random_uniform(dims::Tuple{Integer,Integer}, min::Real, max::Real; seed=nothing) = random_uniform(dims[1], dims[2], min, max; seed=seed)
random_normal(dims::Tuple{Integer,Integer}, mean::Real, std::Real; seed=nothing) = random_normal(dims[1], dims[2], mean, std; seed=seed)

function _binary(name::Symbol, a::Tensor, b::Tensor)
    GC.@preserve a b _wrap_tensor(ccall(_sym(name), Ptr{Cvoid}, (Ptr{Cvoid}, Ptr{Cvoid}), _handle(a, String(name)), _handle(b, String(name))),
                                 String(name))
end

add(a::Tensor, b::Tensor) = _binary(:spiraltorch_tensor_add, a, b)
sub(a::Tensor, b::Tensor) = _binary(:spiraltorch_tensor_sub, a, b)
hadamard(a::Tensor, b::Tensor) = _binary(:spiraltorch_tensor_hadamard, a, b)
matmul(a::Tensor, b::Tensor) = _binary(:spiraltorch_tensor_matmul, a, b)
for op in (:add, :sub, :hadamard, :matmul)
    @eval $op(a::Tensor, b::AbstractMatrix{<:Real}) = $op(a, Tensor(b))
    @eval $op(a::AbstractMatrix{<:Real}, b::Tensor) = $op(Tensor(a), b)
end
Base.:+(a::Tensor, b::Tensor) = add(a, b)
Base.:-(a::Tensor, b::Tensor) = sub(a, b)
Base.:*(a::Tensor, b::Tensor) = matmul(a, b)

function _fused(name::Symbol, a::Tensor, b::Tensor, bias::AbstractVector{<:Real})
    isempty(bias) && error("$(name): empty bias")
    bv = Float32.(collect(bias))
    GC.@preserve a b bv _wrap_tensor(ccall(_sym(name), Ptr{Cvoid}, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cfloat}, Csize_t),
                                          _handle(a, String(name)), _handle(b, String(name)), bv, length(bv)), String(name))
end

"relu(a * b .+ bias'), one bias value per output column, in one library call"
matmul_bias_relu(a::Tensor, b::Tensor, bias::AbstractVector{<:Real}) = _fused(:spiraltorch_tensor_matmul_bias_relu, a, b, bias)
"gelu(a * b .+ bias') in one library call"
matmul_bias_gelu(a::Tensor, b::Tensor, bias::AbstractVector{<:Real}) = _fused(:spiraltorch_tensor_matmul_bias_gelu, a, b, bias)

scale(t::Tensor, v::Real) =
    _wrap_tensor(ccall(_sym(:spiraltorch_tensor_scale), Ptr{Cvoid}, (Ptr{Cvoid}, Cfloat), _handle(t, "tensor_scale"), v), "tensor_scale")
transpose_tensor(t::Tensor) =
    _wrap_tensor(ccall(_sym(:spiraltorch_tensor_transpose), Ptr{Cvoid}, (Ptr{Cvoid},), _handle(t, "tensor_transpose")), "tensor_transpose")
reshape_tensor(t::Tensor, rows::Integer, cols::Integer) =
    _wrap_tensor(ccall(_sym(:spiraltorch_tensor_reshape), Ptr{Cvoid}, (Ptr{Cvoid}, Csize_t, Csize_t), _handle(t, "tensor_reshape"), rows, cols),
                 "tensor_reshape")
row_softmax(t::Tensor) =
    _wrap_tensor(ccall(_sym(:spiraltorch_tensor_row_softmax), Ptr{Cvoid}, (Ptr{Cvoid}, Cint), _handle(t, "tensor_row_softmax"), 0), "tensor_row_softmax")

# ---- runtime ---------------------------------------------------------------------------------------------------
mutable struct Runtime
    handle::Ptr{Cvoid}
end

function Runtime(; worker_threads::Integer=0, thread_name::Union{Nothing,String}=nothing)
    handle = thread_name === nothing ?
        ccall(_sym(:spiraltorch_runtime_new), Ptr{Cvoid}, (Csize_t, Ptr{UInt8}), worker_threads, C_NULL) :
        ccall(_sym(:spiraltorch_runtime_new), Ptr{Cvoid}, (Csize_t, Cstring), worker_threads, thread_name)
    handle == C_NULL && _fail("runtime_new")
    rt = Runtime(handle)
    finalizer(close, rt)
    return rt
end

function Base.close(rt::Runtime)
    if rt.handle != C_NULL
        ccall(_sym(:spiraltorch_runtime_free), Cvoid, (Ptr{Cvoid},), rt.handle)
        rt.handle = C_NULL
    end
    return nothing
end

_rt(rt::Runtime, context) = rt.handle == C_NULL ? error("$context: runtime is closed") : rt.handle
worker_count(rt::Runtime) = Int(ccall(_sym(:spiraltorch_runtime_worker_count), Csize_t, (Ptr{Cvoid},), _rt(rt, "runtime_worker_count")))

function _runtime_binary(name::Symbol, rt::Runtime, a::Tensor, b::Tensor)
    GC.@preserve rt a b _wrap_tensor(ccall(_sym(name), Ptr{Cvoid}, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}), _rt(rt, String(name)),
                                          _handle(a, String(name)), _handle(b, String(name))), String(name))
end

add(rt::Runtime, a::Tensor, b::Tensor) = _runtime_binary(:spiraltorch_runtime_tensor_add, rt, a, b)
sub(rt::Runtime, a::Tensor, b::Tensor) = _runtime_binary(:spiraltorch_runtime_tensor_sub, rt, a, b)
hadamard(rt::Runtime, a::Tensor, b::Tensor) = _runtime_binary(:spiraltorch_runtime_tensor_hadamard, rt, a, b)
matmul(rt::Runtime, a::Tensor, b::Tensor) = _runtime_binary(:spiraltorch_runtime_tensor_matmul, rt, a, b)

function random_uniform(rt::Runtime, rows::Integer, cols::Integer, min::Real, max::Real; seed::Union{Nothing,Integer}=nothing)
    s, has = _seed(seed)
    _wrap_tensor(ccall(_sym(:spiraltorch_runtime_tensor_random_uniform), Ptr{Cvoid}, (Ptr{Cvoid}, Csize_t, Csize_t, Cfloat, Cfloat, UInt64, Bool),
                       _rt(rt, "runtime_tensor_random_uniform"), rows, cols, min, max, s, has), "runtime_tensor_random_uniform")
end

function random_normal(rt::Runtime, rows::Integer, cols::Integer, mean::Real, std::Real; seed::Union{Nothing,Integer}=nothing)
    s, has = _seed(seed)
    _wrap_tensor(ccall(_sym(:spiraltorch_runtime_tensor_random_normal), Ptr{Cvoid}, (Ptr{Cvoid}, Csize_t, Csize_t, Cfloat, Cfloat, UInt64, Bool),
                       _rt(rt, "runtime_tensor_random_normal"), rows, cols, mean, std, s, has), "runtime_tensor_random_normal")
end

# ---- roundtable ------------------------------------------------------------------------------------------------
struct RoundtableSummary
    above::Int
    here::Int
    beneath::Int
    energy_above::Float32
    energy_here::Float32
    energy_beneath::Float32
end

mutable struct _CRoundtableSummary
    above::Csize_t
    here::Csize_t
    beneath::Csize_t
    energy_above::Cfloat
    energy_here::Cfloat
    energy_beneath::Cfloat
end

"""
    roundtable_classify(gradient; above_k, here_k, beneath_k, tolerance=1f-3) -> (assignments, summary)

Bands of a gradient: 0 = above (the largest `above_k` magnitudes), 1 = here (within `tolerance`), 2 = beneath.
"""
function roundtable_classify(gradient::AbstractVector{<:Real}; above_k::Integer, here_k::Integer, beneath_k::Integer, tolerance::Real=1f-3)
    g = Float32.(collect(gradient))
    assignments = Vector{UInt8}(undef, length(g))
    isempty(g) && return assignments, RoundtableSummary(0, 0, 0, 0f0, 0f0, 0f0)
    summary = _CRoundtableSummary(0, 0, 0, 0f0, 0f0, 0f0)
    ok = GC.@preserve g assignments ccall(_sym(:spiraltorch_roundtable_classify), Bool,
                                         (Ptr{Cfloat}, Csize_t, Csize_t, Csize_t, Csize_t, Cfloat, Ptr{UInt8}, Ref{_CRoundtableSummary}),
                                         g, length(g), above_k, here_k, beneath_k, tolerance, assignments, summary)
    ok || _fail("roundtable_classify")
    return assignments, RoundtableSummary(summary.above, summary.here, summary.beneath, summary.energy_above, summary.energy_here, summary.energy_beneath)
end

end # module
