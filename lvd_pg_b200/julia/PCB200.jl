# PCB200.jl — Julia front-end of libpcb200.so for VariationalJuice.jl / LVD-PG.
#
# Defines the reference's own function names on the reference's own types and forwards them
# through `ccall` to the C ABI of include/pcb200.h, so the experiment scripts keep their call
# sites (`loglikelihoods`, `mini_batch_em`, `kld`, `kld_backward`, `sample`, `vectorize_parameters`,
# `update_parameters`).  Device buffers stay `CuArray`s; the library enqueues on CUDA.jl's
# task-local stream.
#
# Written against Julia 1.9+ / CUDA.jl 5 and ProbabilisticCircuits.jl 0.4.  The same ABI is exercised
# by the Python binding in lvd_pg_b200/api.py, which is what the test-suite and the benchmark drive.
module PCB200

using CUDA
using ProbabilisticCircuits
using ProbabilisticCircuits: BitsProbCircuit, SumEdge, BitsInput, BitsSum, BitsMul, dist, isfirst, islast

const libpcb200 = get(ENV, "PCB200_LIB", joinpath(@__DIR__, "..", "libpcb200.so"))
const STATIC_SAMPLE_WORDS = 1 << 20   # capacity of pcb_sample_hard_static's scratch (include/pcb200.h)

struct PcbError <: Exception
    code::Int32
    msg::String
end

function check(code::Int32)
    code == 0 && return
    msg = unsafe_string(ccall((:pcb_last_error, libpcb200), Cstring, ()))
    throw(PcbError(code, msg))
end

# mirror of pcb_circuit_desc
struct CircuitDesc
    num_nodes::UInt32
    num_edges::UInt32
    num_up_layers::UInt32
    num_down_layers::UInt32
    num_input_nodes::UInt32
    num_vars::UInt32
    heap_len::UInt64
    node_kind::Ptr{UInt8}
    node_var::Ptr{UInt32}
    node_num_cats::Ptr{UInt32}
    node_heap_start::Ptr{UInt32}
    node_fixed::Ptr{UInt8}
    up_parent::Ptr{UInt32}
    up_prime::Ptr{UInt32}
    up_sub::Ptr{UInt32}
    up_logp::Ptr{Float32}
    up_tag::Ptr{UInt8}
    up_layer_ends::Ptr{UInt32}
    down2up::Ptr{UInt32}
    down_layer_ends::Ptr{UInt32}
    input_node_ids::Ptr{UInt32}
    heap::Ptr{Float32}
end

"Compiled circuit on the current CUDA device; stands where `CuMetaBitsProbCircuit` stands."
mutable struct PcbCircuit
    handle::Ptr{Cvoid}
    bpc::BitsProbCircuit          # host copy, kept for structure queries and .jpc output
    workspaces::Dict{Int,Ptr{Cvoid}}
    num_inner_params::Int
    num_input_params::Int
end

"Flatten a (host) BitsProbCircuit into the arrays pcb_circuit_create takes."
function PcbCircuit(bpc::BitsProbCircuit; device::Integer = CUDA.deviceid())
    nodes = bpc.nodes
    N = length(nodes)
    kind = Vector{UInt8}(undef, N); var = zeros(UInt32, N); ncat = zeros(UInt32, N)
    hstart = zeros(UInt32, N); fixed = zeros(UInt8, N)
    for (i, n) in enumerate(nodes)
        if n isa BitsInput
            d = dist(n)
            kind[i] = 0; var[i] = n.variable; ncat[i] = d.num_cats; hstart[i] = d.heap_start
            fixed[i] = hasproperty(d, :fixed) && d.fixed ? 1 : 0
        else
            kind[i] = n isa BitsMul ? 1 : 2
        end
    end
    edges = bpc.edge_layers_up.vectors
    E = length(edges)
    parent = UInt32[e.parent_id for e in edges]; prime = UInt32[e.prime_id for e in edges]
    sub = UInt32[e.sub_id for e in edges]
    logp = Float32[e isa SumEdge ? e.logp : 0f0 for e in edges]
    tag = UInt8[e.tag for e in edges]
    up_ends = UInt32.(bpc.edge_layers_up.ends); down_ends = UInt32.(bpc.edge_layers_down.ends)
    down2up = UInt32.(bpc.down2upedge); inputs = UInt32.(bpc.input_node_ids); heap = Float32.(bpc.heap)
    num_vars = maximum(var)
    handle = Ref{Ptr{Cvoid}}(C_NULL)
    GC.@preserve kind var ncat hstart fixed parent prime sub logp tag up_ends down2up down_ends inputs heap begin
        desc = Ref(CircuitDesc(N, E, length(up_ends), length(down_ends), length(inputs), num_vars, length(heap),
            pointer(kind), pointer(var), pointer(ncat), pointer(hstart), pointer(fixed), pointer(parent),
            pointer(prime), pointer(sub), pointer(logp), pointer(tag), pointer(up_ends), pointer(down2up),
            pointer(down_ends), pointer(inputs), pointer(heap)))
        check(ccall((:pcb_circuit_create, libpcb200), Int32, (Ref{CircuitDesc}, Int32, Ref{Ptr{Cvoid}}),
                    desc, device, handle))
    end
    ninner = count(e -> e isa SumEdge, edges)
    ninput = sum(Int(ncat[i]) * (1 - fixed[i]) for i in inputs; init = 0)
    c = PcbCircuit(handle[], bpc, Dict{Int,Ptr{Cvoid}}(), ninner, ninput)
    finalizer(c) do x
        for ws in values(x.workspaces)
            ccall((:pcb_workspace_destroy, libpcb200), Int32, (Ptr{Cvoid},), ws)
        end
        ccall((:pcb_circuit_destroy, libpcb200), Int32, (Ptr{Cvoid},), x.handle)
    end
    c
end
PcbCircuit(pc::ProbCircuit; kw...) = PcbCircuit(BitsProbCircuit(pc); kw...)

stream() = Ptr{Cvoid}(UInt(CUDA.stream().handle))

function workspace(c::PcbCircuit, max_batch::Integer)
    get!(c.workspaces, max_batch) do
        ws = Ref{Ptr{Cvoid}}(C_NULL)
        check(ccall((:pcb_workspace_create, libpcb200), Int32, (Ptr{Cvoid}, UInt32, Int32, Ref{Ptr{Cvoid}}),
                    c.handle, max_batch, 0, ws))
        ws[]
    end
end

import ProbabilisticCircuits: num_parameters, loglikelihoods, update_parameters
num_parameters(c::PcbCircuit) = c.num_inner_params + c.num_input_params

"vectorize_parameters(mbpc, params::CuVector) — src/misc.jl:5-40"
function vectorize_parameters(c::PcbCircuit, params::CuVector{Float32})
    check(ccall((:pcb_get_params_dev, libpcb200), Int32, (Ptr{Cvoid}, CuPtr{Cfloat}, UInt64, Ptr{Cvoid}),
                c.handle, params, length(params), stream()))
    params
end
vectorize_parameters(c::PcbCircuit) = Array(vectorize_parameters(c, CUDA.zeros(Float32, num_parameters(c))))

"update_parameters(mbpc, params::CuVector) — src/misc.jl:73-102"
function update_parameters(c::PcbCircuit, params::CuVector{Float32})
    check(ccall((:pcb_set_params_dev, libpcb200), Int32, (Ptr{Cvoid}, CuPtr{Cfloat}, UInt64, Ptr{Cvoid}),
                c.handle, params, length(params), stream()))
    nothing
end

"loglikelihoods(bpc, data; batch_size) — regularization/reg_likelihood.jl:139-162"
function loglikelihoods(c::PcbCircuit, data::CuMatrix{UInt8}; batch_size = 512)
    n = size(data, 1)
    out = CUDA.zeros(Float32, n)
    ws = workspace(c, batch_size)
    for start in 1:batch_size:n
        b = min(batch_size, n - start + 1)
        check(ccall((:pcb_forward, libpcb200), Int32,
                    (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{UInt8}, CuPtr{UInt8}, UInt64, CuPtr{Int32}, UInt32, UInt32,
                     CuPtr{Cfloat}, Ptr{Cvoid}),
                    c.handle, ws, data, CU_NULL, n, CU_NULL, start, b, pointer(out, start), stream()))
    end
    out
end

"""
mini_batch_em(bpc, data, num_epochs; batch_size, pseudocount, param_inertia, param_inertia_end,
flow_memory, shuffle) — regularization/reg_em.jl:208-336 with soft_reg = 0.
"""
function mini_batch_em(c::PcbCircuit, data::CuMatrix{UInt8}, num_epochs; batch_size, pseudocount,
                       param_inertia, param_inertia_end = param_inertia, flow_memory = 0f0,
                       shuffle = :each_epoch, weights = nothing, verbose = true)
    n = size(data, 1)
    num_batches = n ÷ batch_size
    ws = workspace(c, batch_size)
    ids_cpu = Vector{Int32}(1:n); ids = CuVector{Int32}(ids_cpu)
    do_shuffle() = (ids_cpu .= Int32.(randperm(n)); copyto!(ids, ids_cpu))
    shuffle == :once && do_shuffle()
    Δ = (param_inertia_end - param_inertia) / num_epochs
    rate = iszero(flow_memory) ? 0f0 : max(0f0, 1f0 - (batch_size + pseudocount) / flow_memory)
    lls = Float32[]
    ll_batches = CUDA.zeros(Float32, num_batches)
    wptr = weights === nothing ? CU_NULL : pointer(weights)
    for epoch in 1:num_epochs
        shuffle == :each_epoch && do_shuffle()
        for b in 1:num_batches
            shuffle == :each_batch && do_shuffle()
            check(ccall((:pcb_em_step, libpcb200), Int32,
                        (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{UInt8}, CuPtr{UInt8}, UInt64, CuPtr{Int32}, UInt32, UInt32,
                         CuPtr{Cfloat}, Cfloat, Cfloat, Cfloat, CuPtr{Cfloat}, Ptr{Cvoid}),
                        c.handle, ws, data, CU_NULL, n, pointer(ids, 1 + (b - 1) * batch_size), 1, batch_size,
                        wptr, rate, pseudocount, param_inertia, pointer(ll_batches, b), stream()))
        end
        push!(lls, sum(ll_batches) / batch_size / num_batches)
        param_inertia += Δ
        verbose && println("Mini-batch EM epoch $epoch/$num_epochs; train LL $(lls[end])")
    end
    lls
end

"kld(mbpc, params1, params2) — queries/kld.jl:177-206; params are [S, P] CuMatrix"
function kld(c::PcbCircuit, params1::CuMatrix{Float32}, params2::CuMatrix{Float32})
    S = size(params1, 1)
    out = CUDA.zeros(Float32, S)
    ws = workspace(c, 1)
    check(ccall((:pcb_kld, libpcb200), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Cfloat}, CuPtr{Cfloat}, UInt32, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, ws, params1, params2, S, out, stream()))
    Array(out), ws
end

"kld_backward(mbpc, params1, params2; reuse) — queries/kld.jl:593-649"
function kld_backward(c::PcbCircuit, params1::CuMatrix{Float32}, params2::CuMatrix{Float32}; reuse)
    S, P = size(params1)
    g1 = CUDA.zeros(Float32, S, P); g2 = CUDA.zeros(Float32, S, P)
    check(ccall((:pcb_kld_backward, libpcb200), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Cfloat}, CuPtr{Cfloat}, UInt32, CuPtr{Cfloat}, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, reuse, params1, params2, S, g1, g2, stream()))
    Array(g1), Array(g2)
end

"""
sample(mbpc, params, U_sum, U_leaf) — hard Gumbel-max sampling with caller-supplied uniforms.
U_sum is (kmax, R, S) and U_leaf (cmax, V, S) in Julia's column-major order (the C side reads
[S][R][kmax]); returns x as an (S, V) Int32 matrix of 0-based categories.
"""
function sample(c::PcbCircuit, params::CuMatrix{Float32}, U_sum::CuArray{Float32,3}, U_leaf::CuArray{Float32,3})
    S = size(U_leaf, 3); V = size(U_leaf, 2)
    x = CUDA.zeros(Int32, S, V)
    if S * (V + 2) <= STATIC_SAMPLE_WORDS
        # CUDA.jl's pool owns the device memory: take the entry point that allocates nothing
        check(ccall((:pcb_sample_hard_static, libpcb200), Int32,
                    (Ptr{Cvoid}, CuPtr{Cfloat}, UInt32, CuPtr{Cfloat}, CuPtr{Cfloat}, UInt32, CuPtr{Int32}, Ptr{Cvoid}),
                    c.handle, params, size(params, 1), U_sum, U_leaf, S, x, stream()))
    else
        ws = workspace(c, 1)
        check(ccall((:pcb_sample_hard, libpcb200), Int32,
                    (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Cfloat}, UInt32, CuPtr{Cfloat}, CuPtr{Cfloat}, UInt32, CuPtr{Int32}, Ptr{Cvoid}),
                    c.handle, ws, params, size(params, 1), U_sum, U_leaf, S, x, stream()))
    end
    x
end

end # module
