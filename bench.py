#!/usr/bin/env python
"""Benchmark of the probabilistic-circuit hot path: forward + backward + EM update
(mini-batch EM step) on a seeded synthetic HCLT workload.

    python bench.py --gpus N --steps K --warmup W [--config cfg5|cfg2|...] [--impl reference]

One JSON line on rank 0.  `value` = samples/s of the whole job with data resident in HBM;
`e2e` = the same through the public API with host (pinned) batches copied in every step and the
batch log-likelihood read back; `roofline` = the dominant kernel class against the measured peak;
`cpu_baseline` = the CPU oracle (a restatement of the reference's algorithm) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: (num_vars, latents k, global batch, data rows, description)
    "cfg5": dict(num_vars=3072, k=256, batch=2048, rows=50000, cats=256,
                 desc="HCLT 3072 vars x 256 cats, 256 latents (config 5), mini-batch EM B=2048"),
    "cfg2": dict(num_vars=3072, k=32, batch=512, rows=50000, cats=256,
                 desc="HCLT 3072 vars x 256 cats, 32 latents (config 2), mini-batch EM B=512"),
    "cfg5s": dict(num_vars=384, k=256, batch=2048, rows=8192, cats=256,
                  desc="reduced config 5: first 384 variables, 256 latents, B=2048 (profiling size)"),
    "tiny": dict(num_vars=48, k=32, batch=256, rows=2048, cats=256,
                 desc="tiny smoke workload: 48 variables, 32 latents, B=256"),
}
PSEUDOCOUNT, INERTIA = 0.1, 0.9  # step size 0.1


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "which": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "which": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def build_workload(cfg, device, seed=3):
    from lvd_pg_b200 import synth
    images, fc = synth.image_hclt(cfg["k"], cfg["rows"], 32, 2.0, seed, device,
                                  num_vars=None if cfg["num_vars"] == 3072 else cfg["num_vars"])
    return images, fc


def algorithmic_work(fc, info, B):
    """Per-step algorithmic flops of the dense blocks and bytes of every kernel class, from the
    circuit's own counts (B examples; fp32 = 4 bytes)."""
    n_in = len(fc.input_node_ids)
    N = fc.num_nodes
    Ed = int(info.num_dense_edges)
    Es = int(info.num_inner_params)
    k = fc.meta.get("k", 1)
    dense_nodes = Ed // max(k, 1)           # parents in dense blocks
    work = {
        # three contractions of 2*B*k*k per block: values, child flows, edge statistics
        "dense_fwd": {"flops": 2.0 * B * Ed, "bytes": 4.0 * (B * dense_nodes * 3 + Ed)},
        "dense_bwd_child": {"flops": 2.0 * B * Ed, "bytes": 4.0 * (B * dense_nodes * 6 + Ed)},
        "dense_bwd_edge": {"flops": 2.0 * B * Ed, "bytes": 4.0 * (B * dense_nodes * 4 + 3 * Ed)},
        # leaf values written / leaf flows read once; the parameter tables and the data bytes are small
        # beside them; the leaf statistics are read-modify-written once per step
        "leaf_forward": {"bytes": 4.0 * B * n_in + B * fc.num_vars},
        "leaf_flow": {"bytes": 4.0 * B * n_in + B * fc.num_vars + 8.0 * (fc.num_input_params + n_in)},
        "sparse_up": {"bytes": 4.0 * B * (N - n_in - dense_nodes) * 3},
        "sparse_down": {"bytes": 4.0 * B * (N - 2 * dense_nodes) * 4},
        "em_update": {"bytes": 16.0 * (Es + fc.num_input_params)},
        "w_image": {"bytes": 20.0 * Ed},
    }
    return work


# DRAM bytes per dense block (256 parents x 256 children) at 2048 examples, dram__bytes_read.sum +
# dram__bytes_write.sum of one ncu capture of the largest launches of the 384-variable cut of the
# workload (profiles/dense_tc_kernels_cfg5s.md); traffic grows in proportion to blocks x examples.
NCU_DRAM_BYTES_PER_BLOCK = {"dense_bwd_edge": 2444.6e6 / 287, "dense_bwd_child": 690.4e6 / 55, "dense_fwd": 345.6e6 / 55}


def measured_traffic(kernel_class, info, B, launches_per_step):
    """Per-launch DRAM traffic of a dense class scaled from the ncu capture, or None."""
    per_block = NCU_DRAM_BYTES_PER_BLOCK.get(kernel_class)
    if per_block is None or int(info.num_dense_blocks) == 0 or not launches_per_step:
        return None
    k2 = float(info.num_dense_edges) / float(info.num_dense_blocks)   # edges per block
    return per_block * (k2 / 65536.0) * (B / 2048.0) * int(info.num_dense_blocks) / launches_per_step


def run_cpu_oracle(fc, images_cpu, target_s, rows_hint=None):
    """Time the CPU oracle's EM step on a bounded sample; returns (samples/s, rows, threads, seconds)."""
    from oracle import oracle as orc
    orc.lib()
    threads = orc.num_threads()
    per_row = max(fc.num_edges, 1) * 1.2e-7  # rough single-core seconds per row (fwd + bwd)
    rows = rows_hint or int(max(threads, min(images_cpu.shape[0], threads * max(1, round(target_s / max(per_row, 1e-9))))))
    rows = max(1, min(rows, images_cpu.shape[0]))
    ref = fc.copy()
    data = np.asfortranarray(images_cpu[:rows])
    t0 = time.perf_counter()
    orc.em_step(ref, data, pseudocount=PSEUDOCOUNT, inertia=INERTIA)
    dt = time.perf_counter() - t0
    return rows / dt, rows, threads, dt


def run_cfg4(args):
    """Config 4 (variational path): exact KLD(q || p) + gradient + Adam step, then hard sampling, on
    two HCLTs over 784 binary variables with 64 latents.  One GPU (a single parameter set has no
    batch dimension to shard).  Prints its own JSON line."""
    import torch
    from lvd_pg_b200 import api, synth
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    q, pcirc = synth.config4()
    m = api.CuMetaBitsProbCircuit(q, dev.index)
    theta_q = torch.from_numpy(np.asarray(api.vectorize_parameters(m), np.float32)).to(dev)
    mp = api.CuMetaBitsProbCircuit(pcirc, dev.index)
    theta_p = torch.from_numpy(np.asarray(api.vectorize_parameters(mp), np.float32)).to(dev)
    del mp
    P = int(theta_q.numel())
    adam = api.Adam(m, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8)
    klv = []

    def step():
        kl, reuse = api.kld(m, theta_q, theta_p)
        g1, _ = api.kld_backward(m, reuse=reuse)
        adam.step(theta_q, g1, sign=-1.0)
        klv.append(kl)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index) as clocks:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    # hard sampling of 4096 samples from q with caller-supplied uniforms (seed 5)
    S = 4096
    shp_s, shp_l = api.noise_shapes(m, S)
    g = torch.Generator(device=dev).manual_seed(5)
    u_sum = torch.rand(shp_s, generator=g, device=dev, dtype=torch.float32)
    u_leaf = torch.rand(shp_l, generator=g, device=dev, dtype=torch.float32)
    for _ in range(3):
        x = api.sample(m, theta_q, u_sum, u_leaf)
    torch.cuda.synchronize()
    reps = max(3, args.steps)
    e0.record()
    for _ in range(reps):
        x = api.sample(m, theta_q, u_sum, u_leaf)
    e1.record()
    torch.cuda.synchronize()
    samp_ms = e0.elapsed_time(e1) / reps
    peaks = measured_peaks()
    kld_bytes = 48.0 * P
    samp_bytes = 8.0 * S * (shp_s[1] * shp_s[2] + shp_l[1] * shp_l[2])
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import oracle as orc
        orc.lib()
        tq, tp = theta_q.cpu().numpy().copy(), theta_p.cpu().numpy()
        mm, vv = np.zeros_like(tq), np.zeros_like(tq)
        t0 = time.perf_counter()
        klds, ek = orc.kld(q, tq, tp)
        gr = orc.kld_backward(q, tq, tp, klds, ek)
        orc.adam_step(q, tq, gr["param_grads1"][0], mm, vv, 1)
        cdt = time.perf_counter() - t0
        cpu = {"value": cdt * 1e6, "unit": "us/step", "cores": orc.num_threads(), "kind": "port",
               "sample": "one KLD + gradient + Adam step of the same circuit pair"}
    line = {"metric": "us per KLD+grad+Adam step", "value": us, "unit": "us/step", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "replicas only",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config 4: KLD(q||p) + grad + Adam, HCLT 784 binary vars, 64 latents; then hard sampling S=4096",
                       "params": P, "nodes": q.num_nodes, "edges": q.num_edges, "up_layers": int(m.info.num_up_layers)},
            "kld_last": float(klv[-1][0].item()), "kld_first": float(klv[0][0].item()),
            "roofline": {"bound": "hbm", "achieved": kld_bytes / (us * 1e-6) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": kld_bytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                         "note": "latency-bound: one launch per layer on a single parameter set"},
            "sampling": {"samples_per_s": S / (samp_ms * 1e-3), "ms_per_call": samp_ms, "S": S,
                         "hbm_gbs": samp_bytes / (samp_ms * 1e-3) / 1e9, "hbm_frac": samp_bytes / (samp_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]},
            "clocks": clocks.summary(), "gpu_launches": int(sum(v[1] for v in m.profile_read(reset=True).values()))}
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))


def run_cfg3(args):
    """Config 3 (patch model): forward + backward + EM on 64 independent HCLTs (192 variables,
    128 latents, 256 categories), batch 256 images per circuit, all circuits of a step in flight
    together on their own streams.  With N GPUs the circuits are dealt out 64 / N per rank, no
    collective.  Prints its own JSON line."""
    import torch
    import torch.distributed as dist
    from lvd_pg_b200 import api, synth
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B = 256
    parts = synth.config3(device=dev)
    mine = parts[rank::world]
    circuits = [(api.CuMetaBitsProbCircuit(fc, dev.index), api.DeviceData(data, dev)) for data, fc in mine]
    streams = [torch.cuda.Stream(device=dev) for _ in circuits]
    rng = np.random.default_rng(7)
    n_total = args.warmup + args.steps
    ids = [[torch.from_numpy((rng.permutation(20000)[:B] + 1).astype(np.int32)).to(dev) for _ in circuits] for _ in range(n_total)]
    lls = [torch.zeros(1, device=dev) for _ in circuits]

    def step(i):
        cur = torch.cuda.current_stream(dev)
        for j, (m, dd) in enumerate(circuits):
            streams[j].wait_stream(cur)
            with torch.cuda.stream(streams[j]):
                api.em_step(m, dd, ids[i][j], 1, B, PSEUDOCOUNT, INERTIA, 0.0, None, lls[j])
        for st_ in streams:
            cur.wait_stream(st_)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index) as clocks:
        e0.record()
        for i in range(args.warmup, n_total):
            step(i)
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    launches = sum(sum(v[1] for v in m.profile_read(reset=True).values()) for m, _ in circuits)
    if rank == 0:
        fc0 = mine[0][1]
        line = {"metric": "samples/sec fwd+bwd+EM", "value": 64 * B * args.steps / (ms * 1e-3), "unit": "samples/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "config 3: 64 patch HCLTs (192 vars x 256 cats, 128 latents), B=256 images per circuit, all circuits per step",
                           "circuits": 64, "circuits_per_rank": len(mine), "nodes_per_circuit": fc0.num_nodes,
                           "edges_per_circuit": fc0.num_edges, "parallelism": f"circuits over {world} rank(s), no collective"},
                "train_ll_circuit0": float(lls[0].item()) / B, "clocks": clocks.summary(), "gpu_launches": int(launches)}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default=os.environ.get("PCB_BENCH_CONFIG", "cfg5"))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong: the config's global batch is split over the GPUs (config 5 as stated); "
                         "weak: every GPU takes the config's batch")
    args = ap.parse_args()
    if args.config == "cfg3":
        run_cfg3(args)
        return
    if args.config == "cfg4":
        if int(os.environ.get("RANK", "0")) == 0:
            run_cfg4(args)
        return
    cfg = CONFIGS[args.config]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    Bg = cfg["batch"] * (int(os.environ.get("WORLD_SIZE", "1")) if args.scaling == "weak" else 1)

    if args.impl == "reference":
        # The reference has no CPU implementation of this path and Julia is not installed: the
        # CPU arm is the oracle, a C restatement of the reference's kernels, on all host threads.
        if rank != 0:
            return
        import torch
        from lvd_pg_b200 import synth
        images, fc = build_workload(cfg, "cuda" if torch.cuda.is_available() else "cpu")
        images_cpu = images.cpu().numpy()
        vals, rows, threads = [], 0, 0
        for i in range(args.warmup + args.steps):
            v, rows, threads, dt = run_cpu_oracle(fc, images_cpu, max(2.0, args.cpu_seconds / max(1, args.steps)))
            if i >= args.warmup:
                vals.append((v, dt))
        value = float(np.mean([v for v, _ in vals]))
        line = {"impl": "reference", "metric": "samples/sec fwd+bwd+EM", "value": value, "unit": "samples/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": float(np.mean([dt for _, dt in vals]) * 1e3), "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": cfg["desc"], "bench_config": args.config, "parallelism": "cpu-threads"},
                "cpu_baseline": {"value": value, "unit": "samples/s", "cores": threads, "kind": "port",
                                 "sample": f"{rows} rows per step of the same workload (full circuit)"},
                "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    from lvd_pg_b200 import api

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert Bg % world == 0
    B = Bg // world

    t_setup = time.perf_counter()
    images, fc = build_workload(cfg, dev)
    m = api.CuMetaBitsProbCircuit(fc, local_rank)
    data = api.DeviceData(images, dev)
    if world > 1:
        obj = [api.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(obj, src=0)
        m.attach_comm(obj[0], rank, world)
    rows = data.num_rows
    rng = np.random.default_rng(123)
    n_steps_total = args.warmup + args.steps
    perms = [torch.from_numpy((rng.permutation(rows)[:Bg] + 1).astype(np.int32)) for _ in range(n_steps_total)]
    ids = [p[rank * B:(rank + 1) * B].to(dev) for p in perms]
    ll = torch.zeros(1, device=dev)
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup

    def step(i):
        api.em_step(m, data, ids[i], 1, B, PSEUDOCOUNT, INERTIA, 0.0, None, ll)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    m.profile_read(reset=True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        e0.record()
        for i in range(args.warmup, n_steps_total):
            step(i)
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    launches = sum(v[1] for v in m.profile_read(reset=True).values())
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    value = Bg * args.steps / (ms * 1e-3)
    ll_last = float(ll.item()) / Bg   # the statistics vector (and its log-likelihood slot) is summed over ranks

    # ---- per-kernel-class timing (separate pass, events around every launch) -------------------
    m.profile_enable(True)
    prof_steps = 2
    for i in range(prof_steps):
        step(args.warmup + i % max(1, args.steps))
    prof = m.profile_read(reset=True)
    m.profile_enable(False)
    peaks = measured_peaks()
    work = algorithmic_work(fc, m.info, B)
    classes = {k: v for k, v in prof.items() if v[1] > 0}
    total_prof_ms = sum(v[0] for v in classes.values())
    dom = max(classes, key=lambda k: classes[k][0])
    dom_ms = classes[dom][0] / prof_steps
    w = work.get(dom, {})
    if "flops" in w:
        # dense blocks: 2*B*k*k flops over 4*(3..6)*B*k bytes per block is k/6 .. k/12 flops per byte
        # (21 .. 43 at k = 256, three times that with the TF32 passes counted): far under the ridge of
        # the machine, so the HBM roof is the one that binds.  The tensor-pipe view is kept beside it.
        tfl = w["flops"] / (dom_ms * 1e-3) / 1e12
        achieved = w["bytes"] / (dom_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                "tensor_view": {"achieved": tfl, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": tfl / peaks["tflops"],
                                "note": "algorithmic flops 2*B*E_d of the class; the three TF32 passes are not counted"}}
    else:
        achieved = w.get("bytes", 0.0) / (dom_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": None}
    # the whole step against the HBM roof: algorithmic bytes of every class / timed step
    step_bytes = sum(v.get("bytes", 0.0) for kk, v in work.items() if kk in classes)
    roof["step_hbm"] = {"bytes_per_step": step_bytes, "achieved": step_bytes / (ms / args.steps * 1e-3) / 1e9,
                        "unit": "GB/s", "frac": step_bytes / (ms / args.steps * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    lps = classes[dom][1] / prof_steps
    roof["traffic"] = measured_traffic(dom, m.info, B, lps)
    if roof["traffic"] is not None:
        roof["traffic_unit"] = "bytes per launch (ncu capture of the reduced workload, scaled by blocks x examples)"
        roof["algorithmic_bytes_per_launch"] = w.get("bytes", 0.0) / lps
    # every class against the HBM roof, from its algorithmic bytes and its own event time
    roof["class_hbm_frac"] = {kk: round(work[kk]["bytes"] / (classes[kk][0] / prof_steps * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
                              for kk in classes if kk in work and classes[kk][0] > 0}
    roof.update({"kernel": dom, "kernel_ms_per_step": dom_ms, "launches_per_step": classes[dom][1] / prof_steps,
                 "peak_source": peaks["which"],
                 "class_ms_per_step": {k: round(v[0] / prof_steps, 4) for k, v in classes.items()},
                 "class_share": {k: round(v[0] / total_prof_ms, 4) for k, v in classes.items()}})

    # ---- end to end: host batches in, log-likelihood out ------------------------------------------
    e2e = None
    if not args.no_e2e:
        images_cpu_rows = images.cpu()
        host_batches = []
        for i in range(n_steps_total):
            sel = (perms[i][rank * B:(rank + 1) * B].long() - 1)
            host_batches.append(images_cpu_rows[sel].t().contiguous().pin_memory())  # [V, B] column-major batch
        del images_cpu_rows
        lls = []

        def e2e_step(i):
            batch = host_batches[i].to(dev, non_blocking=True)
            d = api.DeviceData.from_colmajor(batch)
            api.em_step(m, d, None, 1, B, PSEUDOCOUNT, INERTIA, 0.0, None, ll)
            lls.append(float(ll.item()))  # device -> host read of the step's result

        for i in range(args.warmup):
            e2e_step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.warmup, n_steps_total):
            e2e_step(i)
        barrier()
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e = {"value": Bg * args.steps / float(tt.item()), "unit": "samples/s",
               "h2d_bytes_per_step": int(B * fc.num_vars * world), "d2h_bytes_per_step": 4 * world}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, crow, threads, cdt = run_cpu_oracle(fc, images[:4096].cpu().numpy(), args.cpu_seconds)
        cpu_baseline = {"value": v, "unit": "samples/s", "cores": threads, "kind": "port",
                        "sample": f"one EM step on {crow} rows of the same workload (full circuit), {cdt:.1f} s"}

    if rank == 0:
        n_edges = fc.num_edges
        line = {"metric": "samples/sec fwd+bwd+EM", "value": value, "unit": "samples/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": cfg["desc"], "bench_config": args.config, "global_batch": Bg,
                           "parallelism": f"dp{world}", "l2": "inputs (mars+flows) larger than L2" if
                           fc.num_nodes * B * 8 > 126e6 else "working set below L2",
                           "nodes": fc.num_nodes, "edges": n_edges, "sum_edges": int(m.info.num_inner_params),
                           "dense_blocks": int(m.info.num_dense_blocks), "up_layers": int(m.info.num_up_layers),
                           "leaf_params": fc.num_input_params, "setup_s": round(setup_s, 1)},
                "edges_samples_per_s": value * n_edges, "train_ll_last_batch": ll_last,
                "clocks": clocks.summary(), "gpu_launches": int(launches), "roofline": roof}
        if e2e:
            line["e2e"] = e2e
        if cpu_baseline:
            line["cpu_baseline"] = cpu_baseline
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
