#!/usr/bin/env python
"""Benchmark of the hot path on N GPUs of one node.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference        # CPU arm (host cores), same metric and config

One step = one pass of the workload over one batch of seeded synthetic input that is
already resident in HBM. Rank 0 prints one JSON line. Walkers shard across ranks with
no data-path collective (weak scaling: the per-GPU batch is fixed).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

MIB = float(2 ** 20)


# ----------------------------------------------------------------------------- helpers
def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        blob = json.loads(path.read_text())
        return dict(hbm_gbs=float(blob["hbm_gbs"]), bf16_tflops=float(blob["bf16_tflops"]),
                    bf16_tflops_sustained=float(blob.get("bf16_tflops_sustained",
                                                         blob["bf16_tflops"])),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0,
                source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.device_index)],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.split(", ") for r in Path(self.file.name).read_text().splitlines() if r.strip()]
        os.unlink(self.file.name)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[1])); smax.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[5:9]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples taken while the GPU idles between launches would drag the median down:
        # keep the upper half
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:]
        return {"sm_mhz": statistics.median(load), "sm_max_mhz": max(smax),
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus: int):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    if world != n_gpus and world > 1:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}")
    return rank, world, local


def barrier(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, world: int) -> float:
    import torch
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ----------------------------------------------------------------------------- workloads
class AttentionWorkload:
    """The attention benchmark configuration: standalone attention forward + tangent + backward in fp32,
    4096 batch entries x 8 heads x 64 tokens x head dimension 32, no bias, no mask,
    Q,K,V and the tangents/cotangent i.i.d. N(0,1) from a seed."""
    name = "attention fwd+jvp+bwd, B=4096 H=8 L=64 D=32 fp32, no bias, no mask (per GPU)"
    metric = "attention fwd+jvp+bwd batch-entry evals/sec"
    unit = "evals/s"
    B, N, H, D = 4096, 64, 8, 32
    # algorithmic HBM bytes per batch entry (fp32): forward reads q,k,v and writes out,lse;
    # tangent reads q,k,v,out,lse and three tangents and writes one; backward reads
    # q,k,v,out,lse,dout and writes dq,dk,dv.
    launches_per_step = 3

    def __init__(self, rank: int, batch: int | None = None, tf32: bool = False, bias: bool = False):
        import torch
        import hamiltonzero_b200 as hz
        self.hz = hz
        self.torch = torch
        # tf32=True: single-pass TF32 contractions (the arithmetic of the reference's Triton
        # kernels); default: the library's default arithmetic (two-term BF16 split).
        self.mm = hz.HZ_MASK_SQUARE | (hz.HZ_ATTN_TF32 if tf32 else 0)
        if batch:
            self.B = batch
        gen = torch.Generator(device="cuda").manual_seed(2 + rank)
        r = lambda: torch.randn(self.B, self.N, self.H, self.D, device="cuda", generator=gen)
        self.q = r() * self.D ** -0.5
        self.k, self.v, self.qt, self.kt, self.vt, self.do = r(), r(), r(), r(), r(), r()
        # bias=True: the reference-faithful variant with the additive edge bias e [B,N,H,N] read
        # by every pass, its tangent read by the tangent pass and de written by the backward pass
        self.bias = bias
        self.e = self.et = None
        if bias:
            rb = lambda: torch.randn(self.B, self.N, self.H, self.N, device="cuda", generator=gen)
            self.e, self.et = rb(), rb()
        self.out, self.lse = hz.mhsea_fwd(self.q, self.k, self.e, self.v, None, self.mm)
        self.units_per_step = self.B

    def bytes_per_unit(self):
        t = self.N * self.H * self.D * 4
        lse = self.N * self.H * 4
        eb = self.N * self.H * self.N * 4 if self.bias else 0
        return dict(fwd=4 * t + lse + eb, jvp=8 * t + lse + 2 * eb, bwd=8 * t + lse + 2 * eb)

    def step(self):
        hz = self.hz
        self.out, self.lse = hz.mhsea_fwd(self.q, self.k, self.e, self.v, None, self.mm)
        self.tan = hz.mhsea_jvp(self.q, self.k, self.e, self.v, None, self.out, self.lse,
                                self.qt, self.kt, self.et, self.vt, self.mm)
        self.grads = hz.mhsea_bwd(self.q, self.k, self.e, self.v, None, self.lse, self.out,
                                  self.do, need_de=self.bias, mask_mode=self.mm)

    def roofline(self, peaks, ms_per_step, steps):
        ktimes = self.time_dominant_kernel(max(steps, 5))
        top = max(ktimes, key=ktimes.get)
        bytes_unit = self.bytes_per_unit()
        key = {"attn_fwd_kernel": "fwd", "attn_jvp_kernel": "jvp", "attn_bwd_kernel": "bwd"}[top]
        achieved = bytes_unit[key] * self.units_per_step / (ktimes[top] * 1e-3) / 1e9
        return {
            "bound": "hbm", "kernel": top, "achieved": achieved, "peak": peaks["hbm_gbs"],
            "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
            "traffic": None, "per_kernel_ms": ktimes,
            "per_kernel_frac": {k: bytes_unit[{"attn_fwd_kernel": "fwd", "attn_jvp_kernel": "jvp",
                                               "attn_bwd_kernel": "bwd"}[k]] * self.units_per_step
                                / (v * 1e-3) / 1e9 / peaks["hbm_gbs"] for k, v in ktimes.items()},
            "all_passes_frac": sum(bytes_unit.values()) * self.units_per_step
            / (sum(ktimes.values()) * 1e-3) / 1e9 / peaks["hbm_gbs"],
        }

    def time_dominant_kernel(self, iters: int):
        """Average launch duration (ms) of the slowest of the three kernels, by CUDA events
        on the launching stream."""
        torch, hz = self.torch, self.hz
        calls = {
            "attn_fwd_kernel": lambda: hz.mhsea_fwd(self.q, self.k, self.e, self.v, None, self.mm),
            "attn_jvp_kernel": lambda: hz.mhsea_jvp(self.q, self.k, self.e, self.v, None, self.out,
                                                    self.lse, self.qt, self.kt, self.et, self.vt,
                                                    self.mm),
            "attn_bwd_kernel": lambda: hz.mhsea_bwd(self.q, self.k, self.e, self.v, None, self.lse,
                                                    self.out, self.do, need_de=self.bias,
                                                    mask_mode=self.mm),
        }
        times = {}
        for name, fn in calls.items():
            fn(); torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(iters):
                fn()
            e.record(); torch.cuda.synchronize()
            times[name] = s.elapsed_time(e) / iters
        return times

    # end to end: host buffers in, host buffers out
    def e2e_setup(self):
        torch = self.torch
        names = ["q", "k", "v", "qt", "kt", "vt", "do"]
        self.host_in = {n: getattr(self, n).cpu().pin_memory() for n in names}
        self.host_out = [torch.empty_like(self.host_in["q"]).pin_memory() for _ in range(5)]
        self.h2d = sum(t.numel() * 4 for t in self.host_in.values())
        self.d2h = sum(t.numel() * 4 for t in self.host_out)

    def e2e_step(self):
        hz = self.hz
        d = {n: t.to("cuda", non_blocking=True) for n, t in self.host_in.items()}
        out, lse = hz.mhsea_fwd(d["q"], d["k"], None, d["v"], None, self.mm)
        tan = hz.mhsea_jvp(d["q"], d["k"], None, d["v"], None, out, lse, d["qt"], d["kt"], None,
                           d["vt"], self.mm)
        dq, dk, _, dv = hz.mhsea_bwd(d["q"], d["k"], None, d["v"], None, lse, out, d["do"],
                                     need_de=False, mask_mode=self.mm)
        for dst, src in zip(self.host_out, (out, tan, dq, dk, dv)):
            dst.copy_(src, non_blocking=True)

    # CPU arm: the oracle port on a bounded sample of the same workload
    @classmethod
    def cpu_sample(cls, sample_b: int, threads: int):
        import numpy as np
        from concurrent.futures import ThreadPoolExecutor
        from oracle import attention as A
        rng = np.random.default_rng(2)
        f = lambda: rng.standard_normal((sample_b, cls.N, cls.H, cls.D)).astype(np.float32)
        q, k, v, qt, kt, vt, do = (f() for _ in range(7))
        q = q * np.float32(cls.D ** -0.5)

        def one(sl):
            out, lse = A.mhsea_fwd(q[sl], k[sl], None, v[sl], None, dtype=np.float32)
            A.mhsea_jvp(q[sl], k[sl], None, v[sl], None, out, lse, qt[sl], kt[sl], None, vt[sl],
                        dtype=np.float32)
            A.mhsea_bwd(q[sl], k[sl], None, v[sl], None, lse, out, do[sl], dtype=np.float32)

        chunk = max(1, sample_b // (threads * 4))
        slices = [slice(i, min(i + chunk, sample_b)) for i in range(0, sample_b, chunk)]
        pool = ThreadPoolExecutor(max_workers=threads)

        def run():
            list(pool.map(one, slices))
        return run, sample_b


class EnergyWorkload:
    """The configuration the headline metric is quoted on: 64-site Erdos-Renyi
    graph (p = 0.1, seed 7) with a random symmetric 3x3 exchange per edge and a random field
    per node, default model sizes (d_m 1536, ranks 256/256/128) with seeded random arrays,
    16384 walkers per GPU with uniformly random +-1/2 spins; one step = the forward-Laplacian
    local energy (total/exchange/casimir/field) and the spin estimator of every walker."""
    name = ("local energy + spin, 64-site Erdos-Renyi (p=0.1, seed 7) random 3x3 exchange, "
            "default model sizes, 16384 walkers per GPU, n_max=64, fp32")
    metric = "local-energy walker evals/sec at n_max=64"
    unit = "walker evals/s"
    N, B, CHUNK = 64, 16384, 2048

    def __init__(self, rank: int, batch: int | None = None):
        import numpy as np
        import torch
        import hamiltonzero_b200 as hz
        from hamiltonzero_b200 import systems as S
        self.hz, self.torch, self.S = hz, torch, S
        if batch:
            self.B = batch
        frame = S.frame_from_graph(S.erdos_renyi_exchange_graph(self.N, 0.1, seed=7), self.N)
        self.wf_arrays = S.synthetic_wavefunction(0, self.N)
        self.frame_arrays = frame
        self.wf = hz.CompiledWaveFunction(self.wf_arrays)
        self.frame = hz.DeviceEnergyFrame(frame)
        bits = np.random.default_rng(4 + rank).integers(0, 2, (self.B, self.N))
        self.q_host = torch.from_numpy(S.corner_quaternions(bits)).pin_memory()
        self.q = self.q_host.to("cuda")
        self.units_per_step = self.B
        self.launches_per_step = None

    def step(self):
        from hamiltonzero_b200 import walker
        self.out = walker._energy_call(self.wf, self.frame, self.q, self.CHUNK, True)

    def exchange(self):
        """The path's one exchange step (multi-GPU runs): the energy moments of this rank's walkers
        summed over the ranks (src/hamiltonzero/optim/production.py:63-80), one NCCL all-reduce of
        five doubles per step, enqueued behind the step on NCCL's stream (the launching stream does
        not wait for it per step; the timed region ends after every reduction has completed)."""
        from hamiltonzero_b200 import sharding
        total = self.torch.view_as_complex(self.out[1][0])
        self.moments, work = sharding.all_reduce_moments(sharding.local_moments(total), async_op=True)
        return work

    def roofline(self, peaks, ms_per_step, steps):
        """Dominant kernel by accumulated device time in the timed region (per-stage CUDA
        events recorded by the library on the launching stream)."""
        from hamiltonzero_b200 import _lib
        stages = _lib.stage_timing_read(reset=True)
        total_ms = sum(v[0] for v in stages.values()) or 1.0
        top = max(stages, key=lambda k: stages[k][0])
        ms, flops, launches = stages[top]
        achieved = flops / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
        self.launches_per_step = sum(v[2] for v in stages.values()) / max(steps, 1)
        all_flops = sum(v[1] for v in stages.values())
        walkers = min(self.CHUNK, self.B)
        avg_launch_ms = ms / max(launches, 1)
        out = {
            "kernel": top, "avg_launch_ms": avg_launch_ms, "launches": launches,
            "tensor_achieved_tflops": achieved, "tensor_peak_tflops": peaks["bf16_tflops"],
            "tensor_frac": achieved / peaks["bf16_tflops"],
            "frac_of_3xtf32_ceiling": achieved / (peaks["bf16_tflops"] / 6.0),
            "peak_source": peaks["source"],
        }
        if top == "merge_tc_kernel":
            # algorithmic bytes of one launch = the packed jet rows of a level once in and once out
            # (3N Jacobian rows + a value and a Laplacian row per node, d_m floats each), averaged
            # over the levels the kernel runs (the third level up), times the walkers of a launch
            n, row = self.N, 4 * self.wf_arrays.d_m
            levels = range(3, n.bit_length())
            rows = sum(3 * n + 2 * (n >> (l - 1)) + 3 * n + 2 * (n >> l) for l in levels)
            alg_bytes = rows * row / max(len(levels), 1) * walkers
            flops_per_launch = flops / max(launches, 1)
            intensity = flops_per_launch / alg_bytes
            # the roofline's binding ceiling at this arithmetic intensity: memory when
            # intensity * HBM rate is below the tensor peak
            hbm_ceiling_tflops = intensity * peaks["hbm_gbs"] * 1e9 / 1e12
            if hbm_ceiling_tflops < peaks["bf16_tflops"]:
                gbs = alg_bytes / (avg_launch_ms * 1e-3) / 1e9
                out.update({"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": gbs / peaks["hbm_gbs"]})
            else:
                out.update({"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                            "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"]})
            out.update({
                "algorithmic_bytes_per_launch": alg_bytes, "flop_per_byte": intensity,
                "hbm_ceiling_tflops": hbm_ceiling_tflops,
                # dram__bytes_read + dram__bytes_write of merge_tc_kernel from one ncu capture at
                # 256 walkers per launch (levels 3 to 6: 692, 739, 613 and 602 MB; 661.5 MB per
                # launch on average, like avg_launch_ms), scaled to this run's walkers per launch
                "traffic": (661.5e6 / 256) * walkers,
                "traffic_source": "ncu capture at 256 walkers per launch, scaled by walkers per launch"})
        else:
            out.update({"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                        "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"], "traffic": None})
        out.update({
            "stage_share": {k: round(v[0] / total_ms, 4) for k, v in stages.items()},
            "stage_tflops": {k: (round(v[1] / (v[0] * 1e-3) / 1e12, 2) if v[0] > 0 else 0.0)
                             for k, v in stages.items()},
            "algorithmic_gflop_per_walker": all_flops / max(steps, 1) / self.B / 1e9,
            "whole_step_tflops": all_flops / max(steps, 1) / (ms_per_step * 1e-3) / 1e12,
        })
        return out

    def e2e_setup(self):
        self.h2d = self.q_host.numel() * 4
        torch = self.torch
        self.e_host = torch.empty((4, self.B, 2), dtype=torch.float32).pin_memory()
        self.g_host = torch.empty((self.B, 3 * self.N, 2), dtype=torch.float32).pin_memory()
        self.d2h = (self.e_host.numel() + self.g_host.numel()) * 4

    def e2e_step(self):
        from hamiltonzero_b200 import walker
        q = self.q_host.to("cuda", non_blocking=True)
        _lead, energies, _la, _ph, grad = walker._energy_call(self.wf, self.frame, q, self.CHUNK,
                                                              True)
        self.e_host.copy_(energies, non_blocking=True)
        self.g_host.copy_(grad, non_blocking=True)

    @classmethod
    def cpu_sample(cls, sample_b: int, threads: int):
        import numpy as np
        from concurrent.futures import ThreadPoolExecutor
        from hamiltonzero_b200 import systems as S
        from oracle import walker as W
        frame = S.frame_from_graph(S.erdos_renyi_exchange_graph(cls.N, 0.1, seed=7), cls.N)
        wf = S.synthetic_wavefunction(0, cls.N)
        sample_b = max(threads, min(sample_b, 4 * threads))
        q = S.corner_quaternions(np.random.default_rng(4).integers(0, 2, (sample_b, cls.N)))
        per = max(1, sample_b // threads)
        slices = [slice(i, min(i + per, sample_b)) for i in range(0, sample_b, per)]
        pool = ThreadPoolExecutor(max_workers=threads)

        def run():
            list(pool.map(lambda sl: W.local_energy(wf, frame, q[sl], dtype=np.float32), slices))
        return run, sample_b


def context_objects(peaks):
    """Timings of the context compiler's pieces that run on this library's kernels: one
    level-edge attention block at 64 nodes (tuned shape) and the rectangular flash attention of
    the sequence-parallel path (one rank's 512 query rows against 4096 gathered keys, and a
    2048 x 2048 square), CUDA events, L2 flushed between repetitions."""
    import numpy as np
    import torch
    from hamiltonzero_b200 import context as C
    from hamiltonzero_b200 import sequence_parallel as SP

    flush = torch.empty(160 * 1024 * 1024 // 4, device="cuda")

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(); fn(); e.record(); torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        return float(np.median(ts))

    out = {}
    g = torch.Generator(device="cuda").manual_seed(0)
    n, d_c, d_edge = 64, 256, 32
    p = C.init_level_edge_attn(0, d_c, d_edge, alpha_init=0.3, alpha_max=0.5, n_heads=4, attn_dim=128)
    c = torch.randn(n, d_c, device="cuda", generator=g)
    edge = torch.randn(n, n, d_edge, device="cuda", generator=g)
    mask = torch.ones(n, device="cuda")
    out["level_edge_block"] = {"workload": "one LevelEdgeAttn block, 64 nodes, d_c 256, 8 kernel heads of 32, "
                                           "LCA-ALiBi bias (projections and MLPs in torch, attention in hz_mhsea_fwd)",
                               "ms": round(timed(lambda: C.level_edge_attn(p, c, edge, mask, 0)), 4)}
    rect = {}
    for name, (lq, lk) in {"rank_rows_512x4096": (512, 4096), "square_2048": (2048, 2048)}.items():
        h, d = 8, 32
        q = torch.randn(1, lq, h, d, device="cuda", generator=g)
        k = torch.randn(1, lk, h, d, device="cuda", generator=g)
        v = torch.randn(1, lk, h, d, device="cuda", generator=g)
        bias = torch.randn(1, lq, lk, h, device="cuda", generator=g)
        ms = timed(lambda: SP.noncausal_bias_mha(q, k, v, bias))
        byts = 4 * (lq * lk * h + 2 * lk * h * d + 2 * lq * h * d)
        rect[name] = {"Lq": lq, "Lk": lk, "H": h, "D": d, "ms": round(ms, 4),
                      "algorithmic_GBps": round(byts / (ms * 1e-3) / 1e9, 1),
                      "frac_of_hbm": round(byts / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)}
        del q, k, v, bias
    out["rectangular_attention"] = {"op": "hz_mha_rect_fwd (forward, fp32, 3xTF32 mma.sync)", **rect}
    del flush
    torch.cuda.empty_cache()
    return out


def other_configurations(peaks, world):
    """The benchmark configurations other than the headline one, as objects of the default
    line (rank 0): the 8-site chain (256 walkers x 8 replicas of Sz = 0 basis states), the
    periodic 4x4 J1-J2 lattice (4096 walkers) - energy + spin per walker, timed by CUDA events -
    and one cycle of the 256-site lattice configuration on a reduced walker count (sampler sweep
    of 24 steps x 8 replicas with walker_chunk_size = 64, local energy of the cold chain, reverse
    pass with KFAC factor sums, gradient/factor all-reduce); its figures scale linearly with the
    walkers per GPU (4096 in the full configuration)."""
    import numpy as np
    import torch
    import hamiltonzero_b200 as hz
    from hamiltonzero_b200 import _lib, sharding, walker
    from hamiltonzero_b200 import systems as S

    def timed(fn, iters=3):
        fn(); torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record(); torch.cuda.synchronize()
        return s.elapsed_time(e) / iters

    def energy_object(label, graph, n, bits, chunk):
        frame = hz.DeviceEnergyFrame(S.frame_from_graph(graph, n))
        wf = hz.CompiledWaveFunction(S.synthetic_wavefunction(0, n))
        q = torch.from_numpy(S.corner_quaternions(bits)).to("cuda")
        B = q.shape[0] if q.ndim == 3 else int(np.prod(q.shape[:-2]))
        run = lambda: walker._energy_call(wf, frame, q, chunk, True)
        run(); torch.cuda.synchronize()
        _lib.stage_timing_read(reset=True)
        _lib.stage_timing_enable(True)
        run(); torch.cuda.synchronize()
        _lib.stage_timing_enable(False)
        stages = _lib.stage_timing_read(reset=True)
        ms = timed(run)
        flops = sum(v[1] for v in stages.values())
        top = max(stages, key=lambda k: stages[k][0])
        total_ms = sum(v[0] for v in stages.values()) or 1.0
        obj = {"workload": label, "walkers": B, "ms": round(ms, 3),
               "walker_evals_per_s": round(B / (ms * 1e-3), 1),
               "algorithmic_gflop_per_walker": round(flops / B / 1e9, 4),
               "whole_step_tflops": round(flops / (ms * 1e-3) / 1e12, 2),
               "frac_of_3xtf32_ceiling": round(flops / (ms * 1e-3) / 1e12 / (peaks["bf16_tflops"] / 6.0), 4),
               "top_stage": top, "top_stage_share": round(stages[top][0] / total_ms, 3)}
        del wf, frame, q
        torch.cuda.empty_cache()
        return obj

    out = {}
    rng = np.random.default_rng(1)
    bits = np.stack([rng.permutation(np.arange(8) % 2) for _ in range(256 * 8)]).reshape(256, 8, 8)
    out["energy_c1"] = energy_object(
        "8-site open Heisenberg chain, default model sizes, 256 walkers x 8 replicas of Sz = 0 basis states",
        S.chain_graph(8), 8, bits, 2048)
    rng = np.random.default_rng(3)
    bits = np.stack([rng.permutation(np.arange(16) % 2) for _ in range(4096)])
    out["energy_c3"] = energy_object(
        "periodic 4x4 J1-J2 lattice (J1 = 1, J2 = 0.5), default model sizes, 4096 Sz = 0 walkers",
        S.j1j2_square_graph(4), 16, bits, 4096)

    # one cycle of the 256-site configuration on Bw walkers per GPU
    n, Bw, R, steps_mc = 256, 64, 8, 24
    frame_arrays = S.frame_from_graph(S.j1j2_square_graph(16, 1.0, 0.0), n)
    frame = hz.DeviceEnergyFrame(frame_arrays)
    wf = hz.CompiledWaveFunction(S.synthetic_wavefunction(0, n))
    st = hz.mcmc.init_batched_state(5, frame_arrays.mask, Bw, R)
    parts = {}
    holder = {"st": st}

    def sweep():
        holder["st"] = hz.mcmc.run_batched(wf, frame_arrays, holder["st"], steps_mc, 64)
    parts["sampler_sweep_ms"] = timed(sweep, 1)
    cold = hz.mcmc.cold_samples(holder["st"]).contiguous()
    parts["cold_chain_energy_ms"] = timed(lambda: walker._energy_call(wf, frame, cold, 64, False), 2)
    tot = torch.view_as_complex(walker._energy_call(wf, frame, cold, 64, False)[1][0])
    stats = sharding.reduce_moments(sharding.local_moments(tot))
    delta = sharding.centred(tot, stats)
    ca = (2.0 * delta.real / Bw).float().contiguous()
    cp = (2.0 * delta.imag / Bw).float().contiguous()
    res = {}

    def grad():
        res["g"] = wf.vjp(cold, ca, cp, chunk_size=16, factors=True)
    parts["gradient_with_factor_sums_ms"] = timed(grad, 2)
    g, _dq, _la, _ph, fac = res["g"]
    holder["n"] = 0

    def allreduce():
        holder["n"] = sharding.reduce_gradients(g, fac)
    parts["gradient_factor_allreduce_ms"] = timed(allreduce, 2)
    cycle_ms = sum(parts.values())
    evals = (steps_mc + 2) * R * Bw
    out["cycle_c5"] = {
        "workload": "periodic 16x16 Heisenberg lattice (256 sites), default model sizes: 24 replica-exchange "
                    "steps x 8 replicas (walker_chunk_size 64) + local energy of the cold chain + reverse pass "
                    "with KFAC factor sums + gradient/factor all-reduce",
        "walkers_per_gpu": Bw, "walkers_per_gpu_in_the_full_configuration": 4096,
        "scaling_note": "every part is linear in the walkers per GPU except the all-reduce, whose payload "
                        "does not depend on them",
        "parts_ms": {k: round(v, 2) for k, v in parts.items()},
        "cycle_ms": round(cycle_ms, 2),
        "walker_cycles_per_s": round(Bw / (cycle_ms * 1e-3), 2),
        "sampler_value_and_gradient_evals_per_s": round(evals / (parts["sampler_sweep_ms"] * 1e-3), 1),
        "allreduce_floats": int(holder["n"]), "ranks_in_allreduce": world,
        "mean_energy": [round(stats["mean"].real, 4), round(stats["mean"].imag, 4)]}
    return out


WORKLOADS = {"attention_c2": AttentionWorkload, "energy_c4": EnergyWorkload}
DEFAULT_WORKLOAD = "energy_c4"


# ----------------------------------------------------------------------------- arms
def run_reference(args):
    """CPU arm: the oracle port on all host cores, one bounded sample of the workload per step,
    for exactly --steps timed steps after --warmup untimed ones. The reference's own JAX path is
    unavailable on this box (jax, jaxlib and equinox are installed neither in the build
    container nor on the GPU machines, and there is no index to install them from)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    threads = os.cpu_count() or 1
    run, sample = wl.cpu_sample(args.cpu_sample, threads)
    for _ in range(args.warmup):
        run()
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    value = sample / dt
    line = {
        "impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit,
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": wl.name, "sample": f"{sample} of the batch"},
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": threads, "kind": "port",
                         "sample": f"{sample} of the batch per step, NumPy fp32 port of the "
                                   "reference math on a thread pool"},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import __graft_entry__ as entry
    rank, world, local = dist_setup(args.gpus)
    if rank == 0:
        entry.build()
    barrier(world)
    wl_cls = WORKLOADS[args.workload]
    wl = wl_cls(rank, args.batch)
    if args.chunk and hasattr(wl, "CHUNK"):
        wl.CHUNK = args.chunk
    peaks = measured_peaks()

    from hamiltonzero_b200 import _lib
    for _ in range(max(args.warmup, 3)):
        wl.step()
        if world > 1 and hasattr(wl, "exchange"):      # the warm-up step is the timed step
            work = wl.exchange()
            if work is not None:
                work.wait()
    sampler = ClockSampler(local)
    barrier(world)
    _lib.stage_timing_read(reset=True)
    _lib.stage_timing_enable(True)
    sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    pending = []
    for _ in range(args.steps):
        wl.step()
        if world > 1 and hasattr(wl, "exchange"):
            pending.append(wl.exchange())      # enqueued behind the step, on NCCL's stream
    for work in pending:                       # the moments are consumed here: inside the timed region
        if work is not None:
            work.wait()
    end.record()
    barrier(world)
    clocks = sampler.stop()
    _lib.stage_timing_enable(False)
    ms = max_over_ranks(start.elapsed_time(end), world) / args.steps
    value = wl.units_per_step * world / (ms * 1e-3)

    # dominant kernel: per-launch device time by CUDA events on the launching stream
    roofline = wl.roofline(peaks, ms, args.steps)
    attention = None
    if rank == 0 and world == 1 and args.workload == "energy_c4" and not args.no_attention:
        # four arithmetics of the same kernels. Headline: the library default (no flag), the
        # two-term BF16 split with three products per contraction; its distance from the
        # three-term TF32 split's result, and that of the FP16 split, is measured here.
        att = AttentionWorkload(rank)
        hzm = att.hz

        def outputs():
            att.step()
            return [att.out, att.tan, att.grads[0], att.grads[1], att.grads[3]]

        def brief(r, arithmetic):
            return {"arithmetic": arithmetic, "per_kernel_ms": r["per_kernel_ms"],
                    "per_kernel_frac": r["per_kernel_frac"], "all_passes_frac": r["all_passes_frac"]}

        def distance(got, want):
            return {n: float((g - w).abs().max() / w.abs().max())
                    for n, g, w in zip(("out", "tangent", "dq", "dk", "dv"), got, want)}
        att.mm = hzm.HZ_MASK_SQUARE | hzm.HZ_ATTN_TF32X3
        exact = att.roofline(peaks, None, 5)
        want = [t.clone() for t in outputs()]
        att.mm = hzm.HZ_MASK_SQUARE
        attention = att.roofline(peaks, None, 5)
        attention["workload"] = att.name
        attention["arithmetic"] = ("library default (no flag): two-term BF16 split, three products per "
                                   "contraction, fp32 range")
        attention["max_error_vs_tf32x3_of_scale"] = distance(outputs(), want)
        attention["tf32x3_split"] = brief(exact, "three-term TF32 split (flag HZ_ATTN_TF32X3, fp32-faithful)")
        att.mm = hzm.HZ_MASK_SQUARE | hzm.HZ_ATTN_FP16X3
        attention["fp16_split"] = brief(att.roofline(peaks, None, 5),
                                        "two-term FP16 split, three products per contraction (flag "
                                        "HZ_ATTN_FP16X3, operands inside the FP16 range)")
        attention["fp16_split"]["max_error_vs_tf32x3_of_scale"] = distance(outputs(), want)
        att.mm = hzm.HZ_MASK_SQUARE | hzm.HZ_ATTN_TF32
        attention["tf32_single_pass"] = brief(
            att.roofline(peaks, None, 5),
            "one TF32 product per contraction, as the reference's Triton kernels (flag HZ_ATTN_TF32)")
        got = None
        del want, got, att
        torch.cuda.empty_cache()
        # the same three passes with the additive edge bias, as the reference's callers use the op
        att = AttentionWorkload(rank, bias=True)
        with_bias = {}
        for label, flag in (("default_bf16_split", 0), ("fp16_split", hzm.HZ_ATTN_FP16X3),
                            ("tf32x3_split", hzm.HZ_ATTN_TF32X3), ("tf32_single_pass", hzm.HZ_ATTN_TF32)):
            att.mm = hzm.HZ_MASK_SQUARE | flag
            r = att.roofline(peaks, None, 5)
            with_bias[label] = {"per_kernel_ms": r["per_kernel_ms"], "per_kernel_frac": r["per_kernel_frac"],
                                "all_passes_frac": r["all_passes_frac"]}
        attention["with_edge_bias"] = with_bias
        del att
        torch.cuda.empty_cache()
        # a shape the product produces besides the benchmark's: the trunk's 32 kernel heads of
        # dimension 16 at 64 tokens (tiles zero-padded to 32 columns on chip), default arithmetic
        class TrunkHeads(AttentionWorkload):
            name = "attention fwd+jvp+bwd, B=2048 H=32 L=64 D=16 fp32"
            B, N, H, D = 2048, 64, 32, 16
        trunk = {}
        for label, bias in (("no_bias", False), ("with_edge_bias", True)):
            att = TrunkHeads(rank, bias=bias)
            r = att.roofline(peaks, None, 5)
            trunk[label] = {"per_kernel_ms": r["per_kernel_ms"], "per_kernel_frac": r["per_kernel_frac"],
                            "all_passes_frac": r["all_passes_frac"]}
            del att
            torch.cuda.empty_cache()
        attention["trunk_heads_B2048_H32_L64_D16"] = trunk

    # reverse pass (parameter gradients, KFAC factor sums) of the same wavefunction: reported
    # beside the headline, not part of it
    gradient = None
    if rank == 0 and world == 1 and args.workload == "energy_c4" and not args.no_attention:
        nb = min(2048, wl.B)
        qg = wl.q[:nb]
        ca = torch.randn(nb, device="cuda")
        cp = torch.randn(nb, device="cuda")

        def time_vjp(factors):
            wl.wf.vjp(qg, ca, cp, chunk_size=nb, factors=factors)
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(3):
                wl.wf.vjp(qg, ca, cp, chunk_size=nb, factors=factors)
            e.record(); torch.cuda.synchronize()
            return s.elapsed_time(e) / 3
        t_plain, t_fac = time_vjp(False), time_vjp(True)
        gradient = {"op": "hz_logpsi_vjp (all parameter gradients + dq)", "walkers": nb, "walkers_per_pass": nb,
                    "ms": round(t_plain, 3), "walker_vjps_per_s": round(nb / (t_plain * 1e-3), 1),
                    "with_kfac_factor_sums_ms": round(t_fac, 3),
                    "with_kfac_factor_sums_walkers_per_s": round(nb / (t_fac * 1e-3), 1)}
        wl.wf._workspace = None
        torch.cuda.empty_cache()

    # values only (log|psi|, phase) of the same walkers
    logpsi = None
    if rank == 0 and world == 1 and args.workload == "energy_c4" and not args.no_attention:
        nb = min(8192, wl.B)
        wl.wf(wl.q[:nb], chunk_size=4096)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(3):
            wl.wf(wl.q[:nb], chunk_size=4096)
        e.record(); torch.cuda.synchronize()
        t = s.elapsed_time(e) / 3
        logpsi = {"op": "hz_logpsi", "walkers": nb, "ms": round(t, 3),
                  "walkers_per_s": round(nb / (t * 1e-3), 1)}
        wl.wf._workspace = None
        torch.cuda.empty_cache()

    # replica-exchange sampler on the same wavefunction: 256 walkers x 8 replicas, 24 steps per
    # call as in the reference's large-lattice configuration; reported beside the headline
    sampler = None
    if rank == 0 and world == 1 and args.workload == "energy_c4" and not args.no_attention:
        import hamiltonzero_b200 as hz
        Bw, R, steps_mc = 256, 8, 24
        st = hz.mcmc.init_batched_state(11, wl.frame_arrays.mask, Bw, R)
        st = hz.mcmc.run_batched(wl.wf, st, steps_mc)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        st = hz.mcmc.run_batched(wl.wf, st, steps_mc)
        e.record(); torch.cuda.synchronize()
        ms_mc = s.elapsed_time(e)
        grads = (steps_mc + 2) * R * Bw
        sampler = {"op": "hz_mcmc_sweep", "walkers": Bw, "replicas": R, "steps": steps_mc,
                   "ms": round(ms_mc, 2),
                   "value_and_gradient_evals_per_s": round(grads / (ms_mc * 1e-3), 1),
                   "walker_sweeps_per_s": round(Bw / (ms_mc * 1e-3), 2),
                   "local_accept_rate": round(float(st.n_local_accept.sum()) / (Bw * R * st.n_local), 3)}
        del st
        torch.cuda.empty_cache()

    configurations = None
    if rank == 0 and world == 1 and args.workload == "energy_c4" and not args.no_attention:
        wl.wf._workspace = None
        torch.cuda.empty_cache()
        configurations = other_configurations(peaks, 1)

    # the context path's consumers of the attention op (reported beside the headline)
    context_path = None
    if rank == 0 and world == 1 and args.workload == "energy_c4" and not args.no_attention:
        context_path = context_objects(peaks)

    # end to end through the public API with host buffers
    wl.e2e_setup()
    for _ in range(2):
        wl.e2e_step()
    barrier(world)
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(2, min(args.steps, 5))
    s2.record()
    for _ in range(e2e_steps):
        wl.e2e_step()
    e2.record()
    barrier(world)
    e2e_ms = max_over_ranks(s2.elapsed_time(e2), world) / e2e_steps
    e2e = {"value": wl.units_per_step * world / (e2e_ms * 1e-3), "unit": wl.unit,
           "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        run, sample = wl_cls.cpu_sample(args.cpu_sample, threads)
        run()
        t0 = time.perf_counter()
        reps = 2
        for _ in range(reps):
            run()
        dt = (time.perf_counter() - t0) / reps
        cpu_baseline = {"value": sample / dt, "unit": wl.unit, "cores": threads, "kind": "port",
                        "sample": f"{sample} of the batch, NumPy fp32 port on a thread pool"}

    if rank == 0:
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": wl.name, "per_gpu_batch": wl.units_per_step,
                       "walkers_per_pass": getattr(wl, "CHUNK", None),
                       "l2": "per-chunk jet buffers (GBs) and the attention tensors (1.75 GiB) "
                             "exceed the 126 MB L2; no flush needed"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": int(round(wl.launches_per_step * args.steps)), "clocks": clocks,
        }
        if attention is not None:
            line["attention"] = attention
        if gradient is not None:
            line["gradient"] = gradient
        if sampler is not None:
            line["sampler"] = sampler
        if logpsi is not None:
            line["logpsi"] = logpsi
        if configurations is not None:
            line["configurations"] = configurations
        if context_path is not None:
            line["context_path"] = context_path
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=DEFAULT_WORKLOAD)
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch override (profiling)")
    ap.add_argument("--chunk", type=int, default=None,
                    help="walkers per pass of the energy pipeline (memory knob; default 512)")
    ap.add_argument("--cpu-sample", type=int, default=None)
    ap.add_argument("--no-attention", action="store_true",
                    help="skip the attention-op roofline object of the energy workload")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.cpu_sample is None:
        args.cpu_sample = 256 if args.workload == "attention_c2" else 32
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
