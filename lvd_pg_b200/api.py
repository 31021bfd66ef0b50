"""Host-side mirror of the reference's call surface for the probabilistic-circuit hot path.

Same names and argument meaning as the Julia functions they stand for; every one of them
forwards to libpcb200.so through the C ABI of include/pcb200.h:

  CuMetaBitsProbCircuit(pc)             VariationalJuice.jl/src/bits_circuit.jl:5-113
  num_parameters / num_nodes / num_edges                         bits_circuit.jl:119-131
  vectorize_parameters / update_parameters                       src/misc.jl:5-135
  loglikelihoods(bpc, data; batch_size)                          regularization/reg_likelihood.jl:139-162
  mini_batch_em(bpc, data, epochs; batch_size, pseudocount, param_inertia, param_inertia_end,
                flow_memory, shuffle, weights)                   regularization/reg_em.jl:208-336
  full_batch_em                                                  (one step over all rows, inertia 0)
  kld / kld_backward                                             queries/kld.jl:177-206, 593-649
  gumbel_sample (soft) / sample (hard Gumbel-max)                queries/sample.jl:349-383

torch is used for device buffers and streams only.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import _lib
from .circuit import FlatCircuit, PCNode, compile_circuit

ArrayLike = Union[np.ndarray, torch.Tensor]


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class DeviceData:
    """A data matrix [num_rows, num_vars] of uint8 categories resident on the GPU in the
    reference's column-major layout (stored as a contiguous [num_vars, num_rows] tensor)."""

    def __init__(self, data: ArrayLike, device, miss: Optional[ArrayLike] = None):
        self.t = self._put(data, device)
        self.miss = None if miss is None else self._put(miss, device)
        self.num_vars, self.num_rows = int(self.t.shape[0]), int(self.t.shape[1])

    @classmethod
    def from_colmajor(cls, t: torch.Tensor, miss: Optional[torch.Tensor] = None) -> "DeviceData":
        """Wrap a CUDA uint8 tensor that already is [num_vars, num_rows] contiguous."""
        assert t.is_cuda and t.dtype == torch.uint8 and t.is_contiguous() and t.dim() == 2
        self = cls.__new__(cls)
        self.t, self.miss = t, miss
        self.num_vars, self.num_rows = int(t.shape[0]), int(t.shape[1])
        return self

    @staticmethod
    def _put(a: ArrayLike, device) -> torch.Tensor:
        if isinstance(a, np.ndarray):
            a = torch.from_numpy(np.ascontiguousarray(a.T.astype(np.uint8, copy=False)))
        else:
            a = a.to(torch.uint8).t().contiguous()
        return a.to(device, non_blocking=True)


class CuMetaBitsProbCircuit:
    """Compiled circuit on one GPU (cu(BitsProbCircuit) + the flat parameter maps)."""

    def __init__(self, pc: Union[FlatCircuit, PCNode], device: int = 0):
        if not torch.cuda.is_available():
            raise _lib.PcbError(-1, "pcb200 needs a CUDA device; there is no CPU fallback")
        self.fc = pc if isinstance(pc, FlatCircuit) else compile_circuit(pc)
        self.device = torch.device("cuda", device)
        self.lib = _lib.lib()
        h = C.c_void_p()
        desc = self.fc.desc()
        _lib.check(self.lib.pcb_circuit_create(C.byref(desc), device, C.byref(h)))
        self.handle = h
        self.info = _lib.PcbCircuitInfo()
        _lib.check(self.lib.pcb_circuit_get_info(self.handle, C.byref(self.info)))
        self._ws = {}
        self.edge2param = np.zeros(self.fc.num_edges, np.uint32)
        _lib.check(self.lib.pcb_get_edge2param(self.handle, self.edge2param.ctypes.data, self.fc.num_edges))
        self.param2edge = (np.nonzero(self.edge2param)[0] + 1).astype(np.uint32)

    def __del__(self):
        try:
            for ws in self._ws.values():
                self.lib.pcb_workspace_destroy(ws)
            self.lib.pcb_circuit_destroy(self.handle)
        except Exception:
            pass

    def workspace(self, max_batch: int):
        """prep_memory: one workspace per maximal batch size, grown on demand."""
        for cap, ws in self._ws.items():
            if cap >= max_batch:
                return ws
        ws = C.c_void_p()
        _lib.check(self.lib.pcb_workspace_create(self.handle, max_batch, 0, C.byref(ws)))
        self._ws[max_batch] = ws
        return ws

    def free_workspaces(self):
        for ws in self._ws.values():
            self.lib.pcb_workspace_destroy(ws)
        self._ws = {}

    # ---- counters ----
    @property
    def num_inner_params(self) -> int:
        return int(self.info.num_inner_params)

    @property
    def num_input_params(self) -> int:
        return int(self.info.num_input_params)

    @property
    def num_param_groups(self) -> int:
        return int(self.info.num_param_groups)

    def sum_regions(self) -> np.ndarray:
        out = np.zeros(self.fc.num_nodes, np.uint32)
        _lib.check(self.lib.pcb_get_sum_regions(self.handle, out.ctypes.data, out.shape[0]))
        return out

    # ---- parity accessors ----
    def heap(self) -> np.ndarray:
        out = np.zeros(self.fc.heap.shape[0], np.float32)
        _lib.check(self.lib.pcb_get_heap(self.handle, out.ctypes.data, out.shape[0]))
        return out

    def edge_aggr(self) -> np.ndarray:
        out = np.zeros(self.fc.num_edges, np.float32)
        _lib.check(self.lib.pcb_get_edge_aggr(self.handle, out.ctypes.data, out.shape[0]))
        return out

    def _matrix(self, fn, ws, B) -> np.ndarray:
        out = np.zeros((B, self.fc.num_nodes), np.float32, order="F")
        _lib.check(fn(self.handle, ws, out.ctypes.data, out.size))
        return out

    def mars(self, ws, B) -> np.ndarray:
        return self._matrix(self.lib.pcb_get_mars, ws, B)

    def flows(self, ws, B) -> np.ndarray:
        return self._matrix(self.lib.pcb_get_flows, ws, B)

    # ---- launch accounting ----
    def profile_enable(self, on: bool) -> None:
        _lib.check(self.lib.pcb_profile_enable(self.handle, int(on)))

    def profile_read(self, reset: bool = True) -> dict:
        """{kernel class: (milliseconds under event timing, launches)} since the last reset."""
        n = self.lib.pcb_profile_num_classes()
        ms = (C.c_double * n)()
        cnt = (C.c_uint64 * n)()
        _lib.check(self.lib.pcb_profile_read(self.handle, C.cast(ms, C.c_void_p), C.cast(cnt, C.c_void_p), int(reset)))
        return {self.lib.pcb_profile_class_name(i).decode(): (float(ms[i]), int(cnt[i])) for i in range(n)}

    # ---- multi-GPU ----
    def attach_comm(self, unique_id: bytes, rank: int, nranks: int):
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        _lib.check(self.lib.pcb_comm_init(self.handle, C.cast(buf, C.c_void_p), rank, nranks))


    def detach_comm(self):
        """Drop the communicator: later steps run on this GPU alone."""
        _lib.check(self.lib.pcb_comm_destroy(self.handle))


def comm_unique_id() -> bytes:
    buf = (C.c_uint8 * 128)()
    _lib.check(_lib.lib().pcb_comm_unique_id(C.cast(buf, C.c_void_p)))
    return bytes(buf)


def num_parameters(mbpc: CuMetaBitsProbCircuit) -> int:
    return mbpc.num_inner_params + mbpc.num_input_params


def num_nodes(mbpc: CuMetaBitsProbCircuit) -> int:
    return int(mbpc.info.num_nodes)


def num_edges(mbpc: CuMetaBitsProbCircuit) -> int:
    return int(mbpc.info.num_edges)


def vectorize_parameters(mbpc: CuMetaBitsProbCircuit, params: Optional[torch.Tensor] = None):
    """Copy the parameters from `mbpc` to `params` (a CUDA float vector) or return them as numpy."""
    n = num_parameters(mbpc)
    if params is not None:
        assert params.numel() == n and params.is_cuda and params.dtype == torch.float32
        _lib.check(mbpc.lib.pcb_get_params_dev(mbpc.handle, _ptr(params), n, _stream(mbpc.device)))
        return params
    out = np.zeros(n, np.float32)
    _lib.check(mbpc.lib.pcb_get_params(mbpc.handle, out.ctypes.data, n))
    return out


def update_parameters(mbpc: CuMetaBitsProbCircuit, params: ArrayLike) -> None:
    """Copy the parameters from `params` to `mbpc`."""
    n = num_parameters(mbpc)
    if isinstance(params, torch.Tensor) and params.is_cuda:
        assert params.numel() == n and params.dtype == torch.float32 and params.is_contiguous()
        _lib.check(mbpc.lib.pcb_set_params_dev(mbpc.handle, _ptr(params), n, _stream(mbpc.device)))
        return
    p = np.ascontiguousarray(np.asarray(params, dtype=np.float32).reshape(-1))
    assert p.shape[0] == n, f"{n} != {p.shape[0]}"
    _lib.check(mbpc.lib.pcb_set_params(mbpc.handle, p.ctypes.data, n))


def _as_data(mbpc, data) -> DeviceData:
    return data if isinstance(data, DeviceData) else DeviceData(data, mbpc.device)


def forward(mbpc, data, row_ids: Optional[torch.Tensor] = None, row_start: int = 1, B: Optional[int] = None,
            ll_out: Optional[torch.Tensor] = None):
    """eval_circuit on one batch; returns (workspace, B).  row_ids: 1-based int32 CUDA tensor."""
    data = _as_data(mbpc, data)
    if B is None:
        B = int(row_ids.numel()) if row_ids is not None else data.num_rows - (row_start - 1)
    ws = mbpc.workspace(B)
    _lib.check(mbpc.lib.pcb_forward(mbpc.handle, ws, _ptr(data.t), _ptr(data.miss), data.num_rows, _ptr(row_ids),
                                    row_start, B, _ptr(ll_out), _stream(mbpc.device)))
    return ws, B


def backward(mbpc, ws, weights: Optional[torch.Tensor] = None) -> None:
    _lib.check(mbpc.lib.pcb_backward(mbpc.handle, ws, _ptr(weights), _stream(mbpc.device)))


def loglikelihoods(mbpc: CuMetaBitsProbCircuit, data, batch_size: int = 512) -> torch.Tensor:
    """Per-row log-likelihoods, batches of consecutive rows (reg_likelihood.jl:139-162)."""
    data = _as_data(mbpc, data)
    out = torch.empty(data.num_rows, dtype=torch.float32, device=mbpc.device)
    for start in range(0, data.num_rows, batch_size):
        b = min(batch_size, data.num_rows - start)
        forward(mbpc, data, None, start + 1, b, out[start:start + b])
    return out


def em_step(mbpc, data, row_ids=None, row_start=1, B=None, pseudocount=0.1, inertia=0.0, clear_rate=0.0,
            weights=None, ll_sum: Optional[torch.Tensor] = None):
    """Per-batch body of mini_batch_em_with_reg (reg_em.jl:273-301)."""
    data = _as_data(mbpc, data)
    if B is None:
        B = int(row_ids.numel()) if row_ids is not None else data.num_rows - (row_start - 1)
    ws = mbpc.workspace(B)
    _lib.check(mbpc.lib.pcb_em_step(mbpc.handle, ws, _ptr(data.t), _ptr(data.miss), data.num_rows, _ptr(row_ids),
                                    row_start, B, _ptr(weights), clear_rate, pseudocount, inertia, _ptr(ll_sum),
                                    _stream(mbpc.device)))
    return ws


def mini_batch_em(mbpc: CuMetaBitsProbCircuit, data, num_epochs: int, batch_size: int, pseudocount: float,
                  param_inertia: float, param_inertia_end: Optional[float] = None, flow_memory: float = 0.0,
                  shuffle: str = "each_epoch", weights: Optional[torch.Tensor] = None, seed: Optional[int] = None,
                  verbose: bool = False) -> List[float]:
    """mini_batch_em_with_reg with soft_reg = 0 (reg_em.jl:208-336): returns the per-epoch mean
    train log-likelihood.  The last incomplete batch of an epoch is dropped, as in the reference."""
    data = _as_data(mbpc, data)
    n = data.num_rows
    assert batch_size <= n
    if param_inertia_end is None:
        param_inertia_end = param_inertia
    num_batches = n // batch_size
    rng = np.random.default_rng(seed)
    delta = (param_inertia_end - param_inertia) / num_epochs
    ll_epoch = torch.zeros(num_batches, dtype=torch.float32, device=mbpc.device)
    perm_dev = torch.arange(1, n + 1, dtype=torch.int32, device=mbpc.device)

    def do_shuffle():
        perm_dev.copy_(torch.from_numpy((rng.permutation(n) + 1).astype(np.int32)), non_blocking=False)

    if shuffle == "once":
        do_shuffle()
    out = []
    rate = 0.0 if flow_memory == 0 else max(0.0, 1.0 - (batch_size + pseudocount) / flow_memory)
    for epoch in range(num_epochs):
        if shuffle == "each_epoch":
            do_shuffle()
        for b in range(num_batches):
            if shuffle == "each_batch":
                do_shuffle()
            ids = perm_dev[b * batch_size:(b + 1) * batch_size]
            em_step(mbpc, data, ids, 1, batch_size, pseudocount, param_inertia, rate, weights, ll_epoch[b:b + 1])
        ll = float(ll_epoch.sum().item()) / batch_size / num_batches
        _lib.check(mbpc.lib.pcb_circuit_status(mbpc.handle))   # the loop synchronises here anyway (reg_em.jl:303)
        out.append(ll)
        param_inertia += delta
        if verbose:
            print(f"Mini-batch EM epoch {epoch + 1}/{num_epochs}; train LL {ll}")
    return out


def full_batch_em(mbpc: CuMetaBitsProbCircuit, data, num_epochs: int, batch_size: int, pseudocount: float) -> List[float]:
    """Accumulate flows over all rows (in batches), then one update with inertia 0."""
    data = _as_data(mbpc, data)
    out = []
    st = _stream(mbpc.device)
    for _ in range(num_epochs):
        _lib.check(mbpc.lib.pcb_clear_flows(mbpc.handle, 0.0, st))
        lls = torch.empty(data.num_rows, dtype=torch.float32, device=mbpc.device)
        for start in range(0, data.num_rows, batch_size):
            b = min(batch_size, data.num_rows - start)
            ws, _ = forward(mbpc, data, None, start + 1, b, lls[start:start + b])
            backward(mbpc, ws)
        _lib.check(mbpc.lib.pcb_em_update(mbpc.handle, pseudocount, 0.0, st))
        out.append(float(lls.double().mean().item()))
    return out


# ---- KLD ------------------------------------------------------------------------------------------
def _params_matrix(mbpc, p: ArrayLike) -> torch.Tensor:
    """[S, P] parameters as a CUDA tensor in column-major storage (a contiguous [P, S] tensor)."""
    if isinstance(p, np.ndarray):
        p = torch.from_numpy(np.atleast_2d(p).astype(np.float32, copy=False))
    if p.dim() == 1:
        p = p[None, :]
    return p.to(mbpc.device).t().contiguous()


def kld(mbpc: CuMetaBitsProbCircuit, params1: ArrayLike, params2: ArrayLike):
    """Returns (klds[S], reuse): `reuse` is what kld_backward needs (the reference hands back
    the klds / edge_klds matrices for the same purpose, kld.jl:203-205)."""
    p1, p2 = _params_matrix(mbpc, params1), _params_matrix(mbpc, params2)
    S = int(p1.shape[1])
    ws = mbpc.workspace(1)
    out = torch.empty(S, dtype=torch.float32, device=mbpc.device)
    _lib.check(mbpc.lib.pcb_kld(mbpc.handle, ws, _ptr(p1), _ptr(p2), S, _ptr(out), _stream(mbpc.device)))
    return out, (ws, p1, p2, S)


def kld_matrices(mbpc, reuse) -> Tuple[np.ndarray, np.ndarray]:
    """klds [S, N] and edge_klds [S, E] of a kld() call, for parity checks."""
    ws, p1, p2, S = reuse
    klds = np.zeros((S, mbpc.fc.num_nodes), np.float32, order="F")
    _lib.check(mbpc.lib.pcb_get_klds(mbpc.handle, ws, S, klds.ctypes.data))
    ek = torch.zeros(mbpc.fc.num_edges, S, dtype=torch.float32, device=mbpc.device)
    _lib.check(mbpc.lib.pcb_kld_edge_klds(mbpc.handle, ws, _ptr(p1), _ptr(p2), S, _ptr(ek), _stream(mbpc.device)))
    return klds, ek.t().cpu().numpy()


def kld_backward(mbpc: CuMetaBitsProbCircuit, params1=None, params2=None, reuse=None):
    """Gradients of KLD(p1 || p2) w.r.t. the log-parameters of both arguments, [S, P] each."""
    assert reuse is not None, "call kld() first and pass its reuse tuple"
    ws, p1, p2, S = reuse
    P = num_parameters(mbpc)
    g1 = torch.zeros(P, S, dtype=torch.float32, device=mbpc.device)
    g2 = torch.zeros(P, S, dtype=torch.float32, device=mbpc.device)
    _lib.check(mbpc.lib.pcb_kld_backward(mbpc.handle, ws, _ptr(p1), _ptr(p2), S, _ptr(g1), _ptr(g2),
                                         _stream(mbpc.device)))
    return g1.t(), g2.t()


class Adam:
    """Adam on a flat log-parameter vector followed by re-normalisation (sgd/adam.jl:63-127)."""

    def __init__(self, mbpc: CuMetaBitsProbCircuit, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8):
        P = num_parameters(mbpc)
        self.mbpc, self.lr, self.beta1, self.beta2, self.eps = mbpc, lr, beta1, beta2, eps
        self.m = torch.zeros(P, dtype=torch.float32, device=mbpc.device)
        self.v = torch.zeros(P, dtype=torch.float32, device=mbpc.device)
        self.t = 0

    def step(self, theta: torch.Tensor, grad: torch.Tensor, sign: float = -1.0):
        self.t += 1
        grad = grad.contiguous().view(-1)
        _lib.check(self.mbpc.lib.pcb_adam_step(self.mbpc.handle, _ptr(theta), _ptr(grad), _ptr(self.m), _ptr(self.v),
                                               self.t, self.lr, self.beta1, self.beta2, self.eps, sign,
                                               _stream(self.mbpc.device)))


# ---- sampling ---------------------------------------------------------------------------------------
def noise_shapes(mbpc: CuMetaBitsProbCircuit, S: int):
    """Shapes of the uniform buffers `sample` expects: u_sum [S, R, kmax], u_leaf [S, V, cmax]."""
    return ((S, int(mbpc.info.num_sum_regions), int(mbpc.info.max_group_size)),
            (S, mbpc.fc.num_vars, int(mbpc.info.max_num_cats)))


def sample(mbpc: CuMetaBitsProbCircuit, params: ArrayLike, u_sum: ArrayLike, u_leaf: ArrayLike) -> torch.Tensor:
    """Hard Gumbel-max samples x [S, V] (int32, 0-based categories) from caller-supplied uniforms."""
    p = _params_matrix(mbpc, params)
    us = torch.as_tensor(u_sum, dtype=torch.float32).to(mbpc.device).contiguous()
    ul = torch.as_tensor(u_leaf, dtype=torch.float32).to(mbpc.device).contiguous()
    S = int(ul.shape[0])
    shp = noise_shapes(mbpc, S)
    assert tuple(us.shape) == shp[0] and tuple(ul.shape) == shp[1], (us.shape, ul.shape, shp)
    ws = mbpc.workspace(1)
    x = torch.empty(mbpc.fc.num_vars, S, dtype=torch.int32, device=mbpc.device)
    _lib.check(mbpc.lib.pcb_sample_hard(mbpc.handle, ws, _ptr(p), int(p.shape[1]), _ptr(us), _ptr(ul), S, _ptr(x),
                                        _stream(mbpc.device)))
    return x.t()


def sample_static(mbpc: CuMetaBitsProbCircuit, params: torch.Tensor, u_sum: torch.Tensor, u_leaf: torch.Tensor,
                  x_out: torch.Tensor) -> torch.Tensor:
    """`sample` for callers whose memory pool must stay in charge: every buffer, the output
    included, is passed in as a CUDA tensor in the layout the C ABI takes (params [P, Sp]
    contiguous, x_out [V, S] int32) and the library allocates nothing (pcb_sample_hard_static)."""
    S = int(u_leaf.shape[0])
    _lib.check(mbpc.lib.pcb_sample_hard_static(mbpc.handle, _ptr(params), int(params.shape[1]), _ptr(u_sum),
                                               _ptr(u_leaf), S, _ptr(x_out), _stream(mbpc.device)))
    return x_out.t()


def gumbel_sample(mbpc: CuMetaBitsProbCircuit, params: ArrayLike, num_vars: int, par_buffer_size: int,
                  temperature: float, no_gumbel: bool = False, u: Optional[ArrayLike] = None, S: Optional[int] = None):
    """Relaxed top-down sampling: returns input_aggr_params [S, num_vars, par_buffer_size].
    The reference draws its noise in-kernel; here `u` ([S, num_inner_params] uniforms) is passed
    in, or no_gumbel=True selects the noise-free variant."""
    p = _params_matrix(mbpc, params)
    Sp = int(p.shape[1])
    S = S or Sp
    assert num_vars == mbpc.fc.num_vars and par_buffer_size == int(mbpc.info.max_num_cats)
    ud = None
    if not no_gumbel:
        assert u is not None, "pass uniforms `u` or no_gumbel=True"
        ud = torch.as_tensor(u, dtype=torch.float32).to(mbpc.device).t().contiguous()
    ws = mbpc.workspace(1)
    out = torch.empty(par_buffer_size, num_vars, S, dtype=torch.float32, device=mbpc.device)
    _lib.check(mbpc.lib.pcb_sample_soft(mbpc.handle, ws, _ptr(p), Sp, _ptr(ud), temperature, S, _ptr(out),
                                        _stream(mbpc.device)))
    return out.permute(2, 1, 0)
