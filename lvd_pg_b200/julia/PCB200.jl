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
"the same into / from a host vector (the library synchronises and copies itself)"
function vectorize_parameters(c::PcbCircuit, params::Vector{Float32})
    check(ccall((:pcb_get_params, libpcb200), Int32, (Ptr{Cvoid}, Ptr{Cfloat}, UInt64), c.handle, params, length(params)))
    params
end
function update_parameters(c::PcbCircuit, params::Vector{Float32})
    check(ccall((:pcb_set_params, libpcb200), Int32, (Ptr{Cvoid}, Ptr{Cfloat}, UInt64), c.handle, params, length(params)))
    nothing
end

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
        circuit_status(c)   # the loop synchronises here anyway (reg_em.jl:303)
        param_inertia += Δ
        verbose && println("Mini-batch EM epoch $epoch/$num_epochs; train LL $(lls[end])")
    end
    lls
end

"""
kld(mbpc, params1, params2) — queries/kld.jl:177-206; params are [S, P] CuMatrix.  Returns what the
reference returns: `(klds[:, end], (klds_mat, edge_klds_mat))` with host copies of the node values
[S, N] and the edge values [S, E]; the node values also stay in the workspace for `kld_backward`.
"""
function kld(c::PcbCircuit, params1::CuMatrix{Float32}, params2::CuMatrix{Float32})
    S = size(params1, 1)
    out = CUDA.zeros(Float32, S)
    ws = workspace(c, 1)
    check(ccall((:pcb_kld, libpcb200), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Cfloat}, CuPtr{Cfloat}, UInt32, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, ws, params1, params2, S, out, stream()))
    N = length(c.bpc.nodes); E = length(c.bpc.edge_layers_up.vectors)
    klds_mat = Matrix{Float32}(undef, S, N)
    check(ccall((:pcb_get_klds, libpcb200), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, UInt32, Ptr{Cfloat}), c.handle, ws, S, klds_mat))
    edge_klds = CUDA.zeros(Float32, S, E)
    check(ccall((:pcb_kld_edge_klds, libpcb200), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Cfloat}, CuPtr{Cfloat}, UInt32, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, ws, params1, params2, S, edge_klds, stream()))
    Array(out), (klds_mat, Array(edge_klds))
end

"kld_backward(mbpc, params1, params2; reuse) — queries/kld.jl:593-649 (of the last `kld` call on this circuit)"
function kld_backward(c::PcbCircuit, params1::CuMatrix{Float32}, params2::CuMatrix{Float32}; reuse = nothing)
    S, P = size(params1)
    g1 = CUDA.zeros(Float32, S, P); g2 = CUDA.zeros(Float32, S, P)
    check(ccall((:pcb_kld_backward, libpcb200), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Cfloat}, CuPtr{Cfloat}, UInt32, CuPtr{Cfloat}, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, workspace(c, 1), params1, params2, S, g1, g2, stream()))
    Array(g1), Array(g2)
end

# ---- the preallocated forms PCVAE calls (utils/cuda_preallocation.jl:6-78,150-203) ------------------
const prealloc = Dict{Symbol,Any}()

function kld_preallocation(c::PcbCircuit; num_examples)
    P = num_parameters(c)
    prealloc[:kld] = (p1 = CUDA.zeros(Float32, num_examples, P), p2 = CUDA.zeros(Float32, num_examples, P),
                      g1 = CUDA.zeros(Float32, num_examples, P), g2 = CUDA.zeros(Float32, num_examples, P),
                      out = CUDA.zeros(Float32, num_examples))
    nothing
end
kld_free_mem() = (delete!(prealloc, :kld); nothing)

function kld_with_prealloc(c::PcbCircuit, params1, params2; norm_params = false)
    b = prealloc[:kld]
    copyto!(b.p1, params1); copyto!(b.p2, params2)
    S = size(b.p1, 1)
    check(ccall((:pcb_kld, libpcb200), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Cfloat}, CuPtr{Cfloat}, UInt32, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, workspace(c, 1), b.p1, b.p2, S, b.out, stream()))
    Array(b.out)
end

function kld_backward_with_prealloc(c::PcbCircuit; norm_params = false, grad_wrt_logparams = true)
    b = prealloc[:kld]
    S = size(b.p1, 1)
    fill!(b.g1, 0f0); fill!(b.g2, 0f0)
    check(ccall((:pcb_kld_backward, libpcb200), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Cfloat}, CuPtr{Cfloat}, UInt32, CuPtr{Cfloat}, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, workspace(c, 1), b.p1, b.p2, S, b.g1, b.g2, stream()))
    Array(b.g1), Array(b.g2)
end

"""
adam_step!(mbpc, theta, grad, m, v, t; lr, beta1, beta2, eps, sign) — apply_gradients + hard_update_params of
sgd/adam.jl:63-127 on a flat log-parameter vector (sign = -1 descends, as the KLD loop does).
"""
function adam_step!(c::PcbCircuit, theta::CuVector{Float32}, grad::CuVector{Float32}, m::CuVector{Float32},
                    v::CuVector{Float32}, t::Integer; lr = 1f-2, beta1 = 0.9f0, beta2 = 0.999f0, eps = 1f-8, sign = -1f0)
    check(ccall((:pcb_adam_step, libpcb200), Int32,
                (Ptr{Cvoid}, CuPtr{Cfloat}, CuPtr{Cfloat}, CuPtr{Cfloat}, CuPtr{Cfloat}, Int32, Cfloat, Cfloat, Cfloat, Cfloat, Cfloat, Ptr{Cvoid}),
                c.handle, theta, grad, m, v, t, lr, beta1, beta2, eps, sign, stream()))
    theta
end

"One step KLD(q || p) + gradient + Adam on q + re-normalisation as a single (graph-replayed) library call."
function kld_adam_step!(c::PcbCircuit, theta_q::CuVector{Float32}, theta_p::CuVector{Float32}, m::CuVector{Float32},
                        v::CuVector{Float32}, t::Integer, kld_out::CuVector{Float32}; lr = 1f-2, beta1 = 0.9f0,
                        beta2 = 0.999f0, eps = 1f-8)
    check(ccall((:pcb_kld_adam_step, libpcb200), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Cfloat}, CuPtr{Cfloat}, CuPtr{Cfloat}, CuPtr{Cfloat}, Int32, Cfloat, Cfloat, Cfloat, Cfloat, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, workspace(c, 1), theta_q, theta_p, m, v, t, lr, beta1, beta2, eps, kld_out, stream()))
    kld_out
end

"""
gumbel_sample(mbpc, params, num_vars, par_buffer_size; temperature, no_gumbel, u) — queries/sample.jl:349-383.
The reference draws its noise in the kernel; here `u` ([S, num_inner_params] uniforms) is passed in, or
`no_gumbel = true` selects the noise-free variant PCVAE uses.  Returns input_aggr_params [S, V, C] on the host.
"""
function gumbel_sample(c::PcbCircuit, params::CuMatrix{Float32}, num_vars, par_buffer_size; temperature,
                       no_gumbel = false, u = nothing)
    S = size(params, 1)
    out = CUDA.zeros(Float32, S, num_vars, par_buffer_size)
    uptr = no_gumbel ? CU_NULL : pointer(u)
    check(ccall((:pcb_sample_soft, libpcb200), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Cfloat}, UInt32, CuPtr{Cfloat}, Cfloat, UInt32, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, workspace(c, 1), params, S, uptr, temperature, S, out, stream()))
    Array(out)
end
gumbel_sample_with_prealloc(c::PcbCircuit, params; temperature, no_gumbel = false, norm_params = false, u = nothing) =
    gumbel_sample(c, cu(params), Int(maximum(n.variable for n in c.bpc.nodes if n isa BitsInput)),
                  Int(maximum(dist(n).num_cats for n in c.bpc.nodes if n isa BitsInput)); temperature, no_gumbel, u)

# mirror of pcb_evidence (include/pcb200.h)
struct Evidence
    data::CuPtr{UInt8}
    miss::CuPtr{UInt8}
    soft::CuPtr{Cfloat}
    head_mask::CuPtr{Cfloat}
    num_rows::UInt64
    row_ids::CuPtr{Int32}
    row_start::UInt32
    B::UInt32
    soft_reg::Cfloat
    soft_reg_width::UInt32
end

evidence(data::CuMatrix{UInt8}; head_mask = nothing, row_ids = CU_NULL, row_start = 1, B, soft_reg = 0f0, soft_reg_width = 1) =
    Evidence(pointer(data), CU_NULL, CU_NULL, head_mask === nothing ? CU_NULL : pointer(head_mask), size(data, 1),
             row_ids, row_start, B, soft_reg, soft_reg_width)
# a 3-D Float32 array of per-category log-weights [rows, vars, cats] (reg_likelihood.jl:51-91)
evidence(data::CuArray{Float32,3}; head_mask = nothing, row_ids = CU_NULL, row_start = 1, B, kwargs...) =
    Evidence(CU_NULL, CU_NULL, pointer(data), head_mask === nothing ? CU_NULL : pointer(head_mask), size(data, 1),
             row_ids, row_start, B, 0f0, 1)

function forward_ex(c::PcbCircuit, ws, ev::Evidence, ll_out)
    check(ccall((:pcb_forward_ex, libpcb200), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, Ref{Evidence}, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, ws, Ref(ev), ll_out, stream()))
end
function em_step_ex(c::PcbCircuit, ws, ev::Evidence, weights, rate, pseudocount, inertia, ll_sum)
    check(ccall((:pcb_em_step_ex, libpcb200), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, Ref{Evidence}, CuPtr{Cfloat}, Cfloat, Cfloat, Cfloat, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, ws, Ref(ev), weights, rate, pseudocount, inertia, ll_sum, stream()))
end

# the loop of mini_batch_em_with_reg / mini_batch_em_for_multihead_pc over any form of evidence
function em_loop(c::PcbCircuit, data, head_mask, num_epochs; batch_size, pseudocount, soft_reg, soft_reg_width,
                 param_inertia, param_inertia_end, flow_memory, shuffle, weights, verbose)
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
            ev = evidence(data; head_mask, row_ids = pointer(ids, 1 + (b - 1) * batch_size), B = batch_size,
                          soft_reg = Float32(soft_reg), soft_reg_width)
            em_step_ex(c, ws, ev, wptr, rate, pseudocount, param_inertia, pointer(ll_batches, b))
        end
        push!(lls, sum(ll_batches) / batch_size / num_batches)
        circuit_status(c)
        param_inertia += Δ
        verbose && println("Mini-batch EM epoch $epoch/$num_epochs; train LL $(lls[end])")
    end
    lls
end

"""
mini_batch_em_with_reg(bpc, data, num_epochs; ...) — the name and keywords the experiment scripts use
(regularization/reg_em.jl:208-213).  `data` is a UInt8 matrix of categories or a 3-D Float32 array of
per-category log-weights; soft_reg / soft_reg_width regularise the leaves of hard evidence
(reg_likelihood.jl:4-14, reg_flow.jl:3-22).  ent_reg is ignored as in the reference (its entropy step is
commented out, reg_em.jl:294-296); the *_mem / mine / maxe / debug keywords are ignored.
"""
function mini_batch_em_with_reg(c::PcbCircuit, data::Union{CuMatrix{UInt8},CuArray{Float32,3}}, num_epochs;
                                batch_size, pseudocount, soft_reg = 0f0, soft_reg_width = 1, ent_reg = 0f0,
                                param_inertia, param_inertia_end = param_inertia, flow_memory = 0f0,
                                shuffle = :each_epoch, weights = nothing, verbose = true, kwargs...)
    if data isa CuMatrix{UInt8} && iszero(soft_reg)
        return mini_batch_em(c, data, num_epochs; batch_size, pseudocount, param_inertia, param_inertia_end,
                             flow_memory, shuffle, weights, verbose)
    end
    em_loop(c, data, nothing, num_epochs; batch_size, pseudocount, soft_reg, soft_reg_width, param_inertia,
            param_inertia_end, flow_memory, shuffle, weights, verbose)
end

"loglikelihoods_probcat(bpc, data; batch_size) — regularization/reg_likelihood.jl:139-162, hard or soft evidence"
loglikelihoods_probcat(c::PcbCircuit, data::CuMatrix{UInt8}; batch_size = 512, kwargs...) = loglikelihoods(c, data; batch_size)
function loglikelihoods_probcat(c::PcbCircuit, data::CuArray{Float32,3}; batch_size = 512, kwargs...)
    n = size(data, 1)
    out = CUDA.zeros(Float32, n)
    ws = workspace(c, batch_size)
    for start in 1:batch_size:n
        b = min(batch_size, n - start + 1)
        forward_ex(c, ws, evidence(data; row_start = start, B = b), pointer(out, start))
    end
    out
end

"""
per_sample_normalized_flows(mbpc, data[, params]; batch_size) — queries/flow.jl:417-494: an (n, P) CuMatrix
with, per data row, the log of every parameter's share of the flow of its sum node / leaf; `params` is an
(n, P) CuMatrix of log-parameters, one vector per row, or `nothing` for the circuit's own.
"""
function per_sample_normalized_flows(c::PcbCircuit, data::CuMatrix{UInt8}, params = nothing; batch_size = 512, kwargs...)
    n = size(data, 1)
    out = CUDA.zeros(Float32, n, num_parameters(c))
    ws = workspace(c, min(batch_size, n))
    for start in 1:batch_size:n
        b = min(batch_size, n - start + 1)
        check(ccall((:pcb_normalized_flows, libpcb200), Int32,
                    (Ptr{Cvoid}, Ptr{Cvoid}, Ref{Evidence}, CuPtr{Cfloat}, CuPtr{Cfloat}, Ptr{Cvoid}),
                    c.handle, ws, Ref(evidence(data; row_start = start, B = b)),
                    params === nothing ? CU_NULL : pointer(params), out, stream()))
    end
    out
end

"normalize_params(mbpc, params; undo) — misc.jl:448-480, in place on an (S, P) CuMatrix"
function normalize_params(c::PcbCircuit, params::CuMatrix{Float32}; undo = false, kwargs...)
    check(ccall((:pcb_normalize_params, libpcb200), Int32, (Ptr{Cvoid}, CuPtr{Cfloat}, UInt32, Int32, Ptr{Cvoid}),
                c.handle, params, size(params, 1), undo ? 1 : 0, stream()))
    params
end

"The device half of map_pc_parameters (utils/map_params.jl:12-50): params1[:, ids1] = params2[:, ids2]"
function map_pc_parameters!(params1::CuMatrix{Float32}, params2::CuMatrix{Float32}, ids1::CuVector{UInt32}, ids2::CuVector{UInt32})
    check(ccall((:pcb_map_param_columns, libpcb200), Int32,
                (CuPtr{Cfloat}, CuPtr{Cfloat}, UInt32, CuPtr{UInt32}, CuPtr{UInt32}, UInt32, Ptr{Cvoid}),
                params1, params2, size(params1, 1), ids1, ids2, length(ids1), stream()))
    params1
end

"normalized_flows_with_prealloc(mbpc_xz, mbpc_z, data) — utils/cuda_preallocation.jl:287-304, mapping = (ids_z, ids_xz)"
function normalized_flows(c_xz::PcbCircuit, c_z::PcbCircuit, data::CuMatrix{UInt8}, mapping; batch_size = size(data, 1))
    nf = per_sample_normalized_flows(c_xz, data; batch_size)
    pz = CUDA.zeros(Float32, size(data, 1), num_parameters(c_z))
    map_pc_parameters!(pz, nf, mapping[1], mapping[2])
    clamp!(pz, -20f0, 0f0)
    normalize_params(c_z, pz)
end

"""
conditioned_td_prob(mbpc, marked_pc_idx1, marked_pc_idx2, node_probs) — queries/td_prob.jl:277-291; the marks are
Int32 CuVectors over the nodes (`mark_nodes`), node_probs an (S, Z1, Z2) CuArray; returns (S, num_vars, max_cats).
"""
function conditioned_td_prob(c::PcbCircuit, marked1::CuVector{Int32}, marked2::CuVector{Int32},
                             node_probs::CuArray{Float32,3}; num_vars, num_cats)
    S = size(node_probs, 1)
    out = CUDA.zeros(Float32, S, num_vars, num_cats)
    ws = workspace(c, 1)
    check(ccall((:pcb_cond_td_prob, libpcb200), Int32,
                (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Int32}, CuPtr{Int32}, CuPtr{Cfloat}, UInt32, UInt32, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, ws, marked1, marked2, node_probs, S, size(node_probs, 2), out, stream()))
    out
end

"pairwise_MI_chunked(data; num_cats, pseudocount) — utils/information.jl:98-157, as one call on the tensor cores"
function pairwise_MI(data::CuMatrix{UInt8}; num_cats = Int(maximum(data)) + 1, pseudocount = 0.1f0, kwargs...)
    v = size(data, 2)
    mi = CUDA.zeros(Float32, v, v)
    check(ccall((:pcb_pairwise_mi, libpcb200), Int32, (CuPtr{UInt8}, UInt64, UInt32, UInt32, Cfloat, CuPtr{Cfloat}, Ptr{Cvoid}),
                data, size(data, 1), v, num_cats, pseudocount, mi, stream()))
    mi
end

# ---- multi-head circuits (src-jl/multi_head_pc) ---------------------------------------------------------
"""
CuMultiHeadBitsProbCircuit(pcs) — bit_circuit.jl:4-56: the heads under a fake root whose edges carry
tag bit 4 (value 16 of the tag byte), which the library's top-down passes skip.
"""
struct PcbMultiHeadCircuit
    bpc::PcbCircuit
    root_ids::Vector{UInt32}
end
function PcbMultiHeadCircuit(pcs::Vector{<:ProbCircuit}; kw...)
    bpc = BitsProbCircuit(summate(pcs...))
    fake = length(bpc.nodes)
    up = bpc.edge_layers_up.vectors
    for (i, e) in enumerate(up)   # the library reads the tags of the up edges
        if e isa SumEdge && e.parent_id == fake
            up[i] = SumEdge(e.parent_id, e.prime_id, e.sub_id, e.logp, e.tag | 0x10)
        end
    end
    c = PcbCircuit(bpc; kw...)
    roots = zeros(UInt32, length(pcs))
    check(ccall((:pcb_get_head_roots, libpcb200), Int32, (Ptr{Cvoid}, Ptr{UInt32}, UInt64), c.handle, roots, length(roots)))
    PcbMultiHeadCircuit(c, roots)
end

"loglikelihoods(mhbpc, data, head_mask; batch_size) — likelihood.jl:35-66: [rows] with a mask, [rows, heads] without"
function loglikelihoods(m::PcbMultiHeadCircuit, data::CuMatrix{UInt8}, head_mask; batch_size = 512)
    n = size(data, 1); H = length(m.root_ids)
    ws = workspace(m.bpc, batch_size)
    if head_mask === nothing
        out = CUDA.zeros(Float32, n, H)
        tmp = CUDA.zeros(Float32, batch_size, H)
        for start in 1:batch_size:n
            b = min(batch_size, n - start + 1)
            forward_ex(m.bpc, ws, evidence(data; row_start = start, B = b), pointer(tmp))
            out[start:start+b-1, :] .= reshape(view(tmp, 1:b*H), b, H)
        end
        return out
    end
    out = CUDA.zeros(Float32, n)
    for start in 1:batch_size:n
        b = min(batch_size, n - start + 1)
        forward_ex(m.bpc, ws, evidence(data; head_mask, row_start = start, B = b), pointer(out, start))
    end
    out
end
multihead_loglikelihoods_probcat(m::PcbMultiHeadCircuit, data, head_mask; batch_size, kwargs...) =
    loglikelihoods(m, data, head_mask; batch_size)

"mini_batch_em_for_multihead_pc(mhbpc, data, head_mask, num_epochs; ...) — em.jl:1-100"
function mini_batch_em_for_multihead_pc(m::PcbMultiHeadCircuit, data::CuMatrix{UInt8}, head_mask::CuMatrix{Float32},
                                        num_epochs; batch_size, pseudocount, soft_reg = 0f0, soft_reg_width = 1,
                                        param_inertia, param_inertia_end = param_inertia, flow_memory = 0f0,
                                        shuffle = :each_epoch, weights = nothing, verbose = true, kwargs...)
    em_loop(m.bpc, data, head_mask, num_epochs; batch_size, pseudocount, soft_reg, soft_reg_width, param_inertia,
            param_inertia_end, flow_memory, shuffle, weights, verbose)
end

# ---- the pieces of a step and the accessors the reference's tools read ------------------------------
# (the reference runs eval_circuit / flows_circuit / update_params as separate calls in its tests and reads
# edge_aggr afterwards, e.g. for pruning: src/structures/prune.jl:21-31)

"mirror of pcb_circuit_info"
struct CircuitInfo
    num_nodes::UInt32; num_edges::UInt32; num_sum_edges::UInt32; num_up_layers::UInt32
    num_inner_params::UInt32; num_input_params::UInt32; num_param_groups::UInt32; num_dense_blocks::UInt32
    num_sum_regions::UInt32; max_group_size::UInt32; max_num_cats::UInt32
    num_dense_edges::UInt64; device_bytes::UInt64; num_heads::UInt32; reserved::UInt32
end
function circuit_info(c::PcbCircuit)
    info = Ref{CircuitInfo}()
    check(ccall((:pcb_circuit_get_info, libpcb200), Int32, (Ptr{Cvoid}, Ref{CircuitInfo}), c.handle, info))
    info[]
end
version() = ccall((:pcb_version, libpcb200), Int32, ())

"clear_flows: edge_aggr .= 0 (rate = 0) or edge_aggr .*= rate (flow memory), regularization/reg_em.jl:276-284"
clear_flows(c::PcbCircuit, rate::Real = 0) =
    check(ccall((:pcb_clear_flows, libpcb200), Int32, (Ptr{Cvoid}, Cfloat, Ptr{Cvoid}), c.handle, rate, stream()))

"flows_circuit after a forward pass on the same workspace (queries/flow.jl:108-159); weights: per-example CuVector or nothing"
function backward(c::PcbCircuit, ws::Ptr{Cvoid}; weights = nothing)
    wptr = weights === nothing ? CU_NULL : pointer(weights)
    check(ccall((:pcb_backward, libpcb200), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, CuPtr{Cfloat}, Ptr{Cvoid}),
                c.handle, ws, wptr, stream()))
end

"add_pseudocount + aggr_node_flows + update_params + update_input_node_params (reg_em.jl:292-299)"
em_update(c::PcbCircuit; pseudocount::Real, inertia::Real) =
    check(ccall((:pcb_em_update, libpcb200), Int32, (Ptr{Cvoid}, Cfloat, Cfloat, Ptr{Cvoid}),
                c.handle, pseudocount, inertia, stream()))

"edge_aggr in the reference's down-edge order (sum edges filled), after a backward pass or a step"
function edge_aggr(c::PcbCircuit)
    out = zeros(Float32, length(c.bpc.edge_layers_down.vectors))
    check(ccall((:pcb_get_edge_aggr, libpcb200), Int32, (Ptr{Cvoid}, Ptr{Cfloat}, UInt64), c.handle, out, length(out)))
    out
end
"the leaf heap (parameters and flow slots) as bpc.heap lays it out"
function heap(c::PcbCircuit)
    out = zeros(Float32, length(c.bpc.heap))
    check(ccall((:pcb_get_heap, libpcb200), Int32, (Ptr{Cvoid}, Ptr{Cfloat}, UInt64), c.handle, out, length(out)))
    out
end
"edge2param of CuMetaBitsProbCircuit (bits_circuit.jl:39-113): parameter id per up-edge, 0 for product edges"
function edge2param(c::PcbCircuit)
    out = zeros(UInt32, length(c.bpc.edge_layers_up.vectors))
    check(ccall((:pcb_get_edge2param, libpcb200), Int32, (Ptr{Cvoid}, Ptr{UInt32}, UInt64), c.handle, out, length(out)))
    out
end
"sum region (scope class) per node, 0 for non-sum nodes: the R index of the sampling noise"
function sum_regions(c::PcbCircuit)
    out = zeros(UInt32, length(c.bpc.nodes))
    check(ccall((:pcb_get_sum_regions, libpcb200), Int32, (Ptr{Cvoid}, Ptr{UInt32}, UInt64), c.handle, out, length(out)))
    out
end
"mars / flows of the last pass on a workspace as (B, num_nodes) host matrices"
function node_matrix(sym::Symbol, c::PcbCircuit, ws::Ptr{Cvoid}, B::Integer)
    out = zeros(Float32, B, length(c.bpc.nodes))
    if sym === :mars
        check(ccall((:pcb_get_mars, libpcb200), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cfloat}, UInt64), c.handle, ws, out, length(out)))
    else
        check(ccall((:pcb_get_flows, libpcb200), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cfloat}, UInt64), c.handle, ws, out, length(out)))
    end
    out
end
get_mars(c::PcbCircuit, ws::Ptr{Cvoid}, B::Integer) = node_matrix(:mars, c, ws, B)
get_flows(c::PcbCircuit, ws::Ptr{Cvoid}, B::Integer) = node_matrix(:flows, c, ws, B)

# launch accounting: what the reference's debug = true prints with CUDA.@time (queries/likelihood.jl:86-92)
profile_enable(c::PcbCircuit, on::Bool) =
    check(ccall((:pcb_profile_enable, libpcb200), Int32, (Ptr{Cvoid}, Int32), c.handle, on ? 1 : 0))
"Dict(kernel class => (milliseconds under event timing, launches)) since the last reset"
function profile_read(c::PcbCircuit; reset::Bool = true)
    n = ccall((:pcb_profile_num_classes, libpcb200), Int32, ())
    ms = zeros(Float64, n); cnt = zeros(UInt64, n)
    check(ccall((:pcb_profile_read, libpcb200), Int32, (Ptr{Cvoid}, Ptr{Float64}, Ptr{UInt64}, Int32), c.handle, ms, cnt, reset ? 1 : 0))
    Dict(unsafe_string(ccall((:pcb_profile_class_name, libpcb200), Cstring, (Int32,), i - 1)) => (ms[i], Int(cnt[i])) for i in 1:n)
end

"Waits for the device and throws if a kernel of this circuit gave up a bounded wait (call where the loop synchronises)."
circuit_status(c::PcbCircuit) = check(ccall((:pcb_circuit_status, libpcb200), Int32, (Ptr{Cvoid},), c.handle))

"""
selftest_wait_limit(device = 0; polls = 2^16) — runs the bounded mbarrier wait of the tensor-core kernels on a barrier
nothing arrives at: returns (status, after, ms, production_polls); status == 1 and after == 2 mean that the wait gave
up, reported and let the kernel return.  ms * production_polls / polls is how long a lost signal holds a kernel.
"""
function selftest_wait_limit(device::Integer = 0; polls::Integer = 1 << 16)
    status = Ref{Int32}(-1); after = Ref{Int32}(-1); ms = Ref{Float32}(0); prod = Ref{UInt32}(0)
    check(ccall((:pcb_selftest_wait_limit, libpcb200), Int32,
                (Int32, UInt32, Ref{Int32}, Ref{Int32}, Ref{Float32}, Ref{UInt32}), device, polls, status, after, ms, prod))
    (status = status[], after = after[], ms = ms[], production_polls = prod[])
end

# ---- multi-GPU: one NCCL communicator per process (no counterpart in the reference) ------------------
function comm_unique_id()
    id = zeros(UInt8, 128)
    check(ccall((:pcb_comm_unique_id, libpcb200), Int32, (Ptr{UInt8},), id))
    id
end
comm_init(c::PcbCircuit, id::Vector{UInt8}, rank::Integer, nranks::Integer) =
    check(ccall((:pcb_comm_init, libpcb200), Int32, (Ptr{Cvoid}, Ptr{UInt8}, Int32, Int32), c.handle, id, rank, nranks))
comm_destroy(c::PcbCircuit) = check(ccall((:pcb_comm_destroy, libpcb200), Int32, (Ptr{Cvoid},), c.handle))
"enabled = false skips the step's collectives (to time what they leave exposed; not for training)"
comm_set_enabled(c::PcbCircuit, enabled::Bool) =
    check(ccall((:pcb_comm_set_enabled, libpcb200), Int32, (Ptr{Cvoid}, Int32), c.handle, enabled ? 1 : 0))
"throws when NCCL reports an asynchronous error of the communicator (a lost peer, a network fault)"
comm_poll(c::PcbCircuit) = check(ccall((:pcb_comm_poll, libpcb200), Int32, (Ptr{Cvoid},), c.handle))
"""
comm_wait(c; timeout_s, stream) — the bounded counterpart of CUDA.synchronize() after steps with a collective:
returns when the stream has drained; on an NCCL error or after `timeout_s` the communicator is aborted and an
error thrown (call comm_destroy before the next step).
"""
comm_wait(c::PcbCircuit; timeout_s::Real = 60, stream = stream()) =
    check(ccall((:pcb_comm_wait, libpcb200), Int32, (Ptr{Cvoid}, Ptr{Cvoid}, UInt32), c.handle, stream,
                round(UInt32, 1000 * timeout_s)))
"ends the communicator without waiting for its collectives"
comm_abort(c::PcbCircuit) = check(ccall((:pcb_comm_abort, libpcb200), Int32, (Ptr{Cvoid},), c.handle))

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
