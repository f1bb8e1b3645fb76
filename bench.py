#!/usr/bin/env python
"""Benchmark of the joint-attention hot path (hd128, S = 4608: 512 text + 64x64 image tokens).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the hot path over one batch: fused QK-RMSNorm + 4-axis RoPE, then
joint attention, through the C ABI. Work counted per step: 4 * B * H * S^2 * D flops (QK^T
and PV only; norm, RoPE and softmax are not counted).

N = 1: B = 1, 32 heads (the 1024px generation step). N > 1 (one process per GPU under
torchrun): batch N with the 32 heads sharded 32/N per GPU, so every GPU still owns 32
(batch, head) units - weak scaling, no collective on the data path.

`value` is device-timed with inputs resident in HBM; `e2e` is the same step through the
host-buffer entry point with pinned host tensors (H2D of Q, K, V and D2H of O inside the
timed region). `roofline` times the attention kernel alone. `cpu_baseline` is the fp32 host
restatement (oracle/) on a bounded head sample; `reference_kernel` is a short run of the
reference's own CUDA kernels, rebuilt for sm_100a (oracle/_ref), on the same GPU in the same
run. `--impl reference` runs those kernels as the whole measurement on the same workload.

Other workloads (--workload): the long shapes with the sequence sharded over the GPUs
(*_seqpar) or with the heads sharded (*_heads), and the batch-4 step with heads sharded; these
are strong-scaling jobs and print the same line without the roofline, e2e and CPU legs.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# The head exchange drives one copy stream per destination rank; each needs a hardware queue of its
# own (see f2k_hx_exchange_in_copy). Has to be in the environment before CUDA is initialised.
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

import numpy as np  # noqa: E402
import torch  # noqa: E402

HEADLINE_WORKLOAD = "s4608 joint attention (512 text + 64x64 image tokens, hd128), batch 1, 32 heads"
METRIC = "joint_attn_tflops"
UNIT = "TFLOP/s"
FALLBACK_PEAK_TFLOPS = 1590.0
STRONG_SECTION_LIMIT_S = 420
# DRAM bytes (read + write) of one attention-kernel launch at S=4608, B=1, H=32, as counted by one
# ncu capture (dram__bytes_read.sum + dram__bytes_write.sum); algorithmic minimum 151.0 MB.
ATTN_DRAM_TRAFFIC_BYTES = 129.9e6


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="s4608",
                    choices=["s4608", "s8704_seqpar", "s16896_seqpar", "s4608_b4_heads", "s8704_heads", "s16896_heads",
                             "s8704_hx", "s16896_hx", "s8704_hxfused", "s16896_hxfused", "s8704_hxce", "s16896_hxce"],
                    help="s4608: the headline shape (heads sharded over the GPUs, batch grows with N). *_seqpar: the "
                         "long shapes with the sequence sharded over the GPUs (strong scaling, K/V pulled over NVLink "
                         "under the kernel). *_heads: a fixed job with its 32 heads sharded 32/N per GPU (strong scaling). "
                         "*_hx: sequence sharded outside, heads sharded inside (head exchange by a scatter kernel in front "
                         "of the attention kernel); *_hxfused: the exchange on the attention kernel's spare warps; "
                         "*_hxce: copy engines deliver under the attention kernel")
    ap.add_argument("--no-overlap", action="store_true", help="seqpar: start the kernel only after all K/V pulls")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the timed CPU leg")
    ap.add_argument("--no-reference-kernel", action="store_true",
                    help="skip the short leg that times the reference's rebuilt kernels beside ours (N = 1)")
    ap.add_argument("--skip-denoise-step", action="store_true", help="skip the 32-call CUDA-graph leg (N = 1)")
    ap.add_argument("--skip-sustained", action="store_true", help="skip the seconds-long back-to-back leg (N = 1)")
    ap.add_argument("--sustained-seconds", type=float, default=2.5)
    ap.add_argument("--skip-strong-scaling", action="store_true",
                    help="N > 1: skip the fixed jobs (heads / sequence / head exchange) after the headline legs")
    ap.add_argument("--strong-jobs", default="",
                    help="comma-separated subset of the strong-scaling jobs to run (default: all)")
    ap.add_argument("--skip-e2e", action="store_true",
                    help="skip the host-buffer leg (for short profiler captures; the line then has e2e null)")
    return ap.parse_args()


def measured_peak(key="bf16_tflops"):
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            d = json.loads(f.read_text())
            what = "cuBLAS burst" if key == "bf16_tflops" else "cuBLAS back to back for seconds"
            return float(d[key]), f"measured {key} ({what}, MEASURED_PEAKS.json)"
        except Exception:
            pass
    if key == "bf16_tflops":
        return FALLBACK_PEAK_TFLOPS, "fallback 1590 TFLOP/s (MEASURED_PEAKS.json absent)"
    return 1400.0, "fallback 1400 TFLOP/s sustained (MEASURED_PEAKS.json absent)"


class ClockSampler:
    """SM clock and throttle reasons of one GPU, read through NVML every few milliseconds by a
    thread of this process while the timed regions run (reading only; nothing is set)."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, device: int, period_s: float = 0.004):
        import threading
        self.samples, self.mask, self.max_mhz, self.err = [], 0, None, None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons

            def poll():
                while not self._stop.is_set():
                    try:
                        self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        self.mask |= int(reasons(h))
                    except Exception as exc:
                        self.err = str(exc)
                        return
                    time.sleep(period_s)

            self._thread = threading.Thread(target=poll, daemon=True)
            self._thread.start()
        except Exception as exc:
            self.err = f"NVML unavailable: {exc}"

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [self.err or "no samples"]}
        top = max(self.samples)
        load = [x for x in self.samples if x >= 0.6 * top]       # samples taken while kernels ran
        return {"sm_mhz": statistics.median(load), "sm_min_mhz": min(load), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(n for bit, n in self.REASONS.items() if self.mask & bit), "samples": len(self.samples)}

    def bins(self, width_mhz: int = 100):
        """Share of the samples per SM-clock bin (lower edge in MHz)."""
        if not self.samples:
            return {}
        out = {}
        for x in self.samples:
            k = str(int(x // width_mhz) * width_mhz)
            out[k] = out.get(k, 0) + 1
        return {k: round(v / len(self.samples), 3) for k, v in sorted(out.items(), key=lambda kv: int(kv[0]))}


def dev_bf16(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).cuda()


def pinned(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).pin_memory()


def time_region(fn, steps, stream):
    """Milliseconds per step of `fn` called `steps` times, CUDA events on the launching stream."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def make_rank_problem(n_gpus: int, rank: int):
    """Host tensors of this rank: batch n_gpus, heads [rank*32/n, (rank+1)*32/n)."""
    from f2k_cuda_b200.inputs import SEED_BASE, Workload, make_problem
    heads = 32 // n_gpus
    w = Workload("s4608", n_gpus, 512, ((64, 64),), seed=SEED_BASE + 1)
    # every rank draws its own heads: same distribution, rank-dependent seed keeps it cheap
    wl = Workload("s4608", n_gpus, 512, ((64, 64),), n_heads=heads, seed=SEED_BASE + 1 + 1000 * rank)
    return w, make_problem(wl)


def cpu_baseline(problem, tabs, flops_per_head):
    """fp32 host restatement (oracle/, OpenMP) on a bounded sample of heads of the same workload."""
    import oracle
    orc = oracle.load_oracle()
    p = problem
    D = p.w.head_dim
    H = p.q_img.shape[2]

    def run(h0, h1):
        t0 = time.perf_counter()
        prep = {}
        for name, x, g, (cos, sin), seq in (("q_txt", p.q_txt, p.gammas[0], tabs[0:2], p.w.seq_txt),
                                            ("k_txt", p.k_txt, p.gammas[1], tabs[0:2], p.w.seq_txt),
                                            ("q_img", p.q_img, p.gammas[2], tabs[2:4], p.w.seq_img),
                                            ("k_img", p.k_img, p.gammas[3], tabs[2:4], p.w.seq_img)):
            xs = np.ascontiguousarray(x[:1, :, h0:h1])
            n = xs.shape[2]
            y = orc.rmsnorm_bf16(xs.reshape(-1, D), g, 1e-6)
            pos = ((np.arange(seq * n) // n) % seq).astype(np.int32)
            prep[name] = orc.rope_bf16(y, cos, sin, pos, seq).reshape(1, seq, n, D)
        q = np.concatenate([prep["q_txt"], prep["q_img"]], 1)
        k = np.concatenate([prep["k_txt"], prep["k_img"]], 1)
        v = np.concatenate([p.v_txt[:1, :, h0:h1], p.v_img[:1, :, h0:h1]], 1)
        orc.attention_f32(q, k, v)
        return time.perf_counter() - t0

    t1 = run(0, 1)                                   # calibration: one head
    n = int(max(1, min(H, 15.0 / max(t1, 1e-3))))   # about 15 s of CPU work
    t = run(0, n)
    return {"value": n * flops_per_head / t / 1e12, "unit": UNIT, "cores": orc.threads, "kind": "port",
            "sample": f"batch element 0, heads 0..{n - 1} of {H} (S=4608): QK-norm + RoPE + fp32 attention, {t:.1f} s"}


def denoise_step_leg(d, dg, dtab, o_t, o_i, B, St, Si, H, D, stream, flops_per_call, guidance):
    """The attention calls of one denoise step (reference: 8 DoubleStreamBlock + 24 SingleStreamBlock
    forwards per model forward, flux_transformer.cu:412-439; two model forwards per step under
    classifier-free guidance, tools/serve.cu:563-566), captured once as a CUDA graph and replayed:
    time per step and per call without per-call launch overhead. Every call of a kind reads the same
    input tensors (memory), which does not change its work."""
    from f2k_cuda_b200.step import DoubleCall, SingleCall, StepAttention
    step = StepAttention(B, St, Si, H, D)
    if not step.ok():
        return {"unavailable": step.last_error()}
    qc, kc, vc = (torch.cat([d[i], d[i + 3]], 1).contiguous() for i in range(3))
    oc = torch.empty_like(qc)
    tab_c = [torch.cat([dtab[0], dtab[2]]).contiguous(), torch.cat([dtab[1], dtab[3]]).contiguous()]
    one_pass = ([DoubleCall(*d, o_t, o_i)] * 8, [SingleCall(qc, kc, vc, oc)] * 24)
    passes = [one_pass] * (2 if guidance else 1)
    graph, calls = step.capture(passes, dg, dtab, tab_c)
    for _ in range(2):
        graph.replay()
    reps = 5
    ms = time_region(graph.replay, reps, stream)
    if step.device_status() != 0:
        raise RuntimeError("attention kernel reported a device-side error in the denoise-step leg")
    return {"calls": calls, "ms_per_step": ms, "ms_per_call": ms / calls,
            "value": calls * flops_per_call / (ms * 1e-3) / 1e12, "unit": UNIT,
            "launch": f"one CUDA graph of {2 * calls} kernels, replayed", "steps": reps,
            "what": ("classifier-free guidance, two model forwards: 2 x " if guidance else "") +
                    "(8 joint calls (512 + 4096 tokens) + 24 single-stream calls (4608 tokens)), fused prologue each"}


def _headline_line(args, world, flops, ms, ms_attn, ms_e2e, e2e_steps, d, o_t, o_i, clocks, B, H, St, Si, D):
    peak, peak_src = measured_peak()
    achieved = flops / (ms_attn * 1e-3) / 1e12
    in_bytes = sum(x.numel() * 2 for x in d)
    out_bytes = o_t.numel() * 2 + o_i.numel() * 2
    line = {
        "metric": METRIC, "value": world * flops / (ms * 1e-3) / 1e12, "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": HEADLINE_WORKLOAD if world == 1 else
                               "s4608 joint attention (512 text + 64x64 image tokens, hd128), "
                               f"batch {B}, {H} heads per GPU (heads sharded)",
                   "step": "fused QK-RMSNorm + 4-axis RoPE + non-causal attention, one call",
                   "flops_per_step_per_gpu": flops, "seq": St + Si, "head_dim": D,
                   "l2": "inputs + outputs + workspace of a step exceed the 126 MB L2 (226 MB)",
                   "parallelism": f"heads{world}" if world > 1 else "single"},
        "per_gpu_tflops": flops / (ms * 1e-3) / 1e12,
        "pct_of_peak": 100.0 * flops / (ms * 1e-3) / 1e12 / peak,
        "roofline": {"bound": "tensor", "kernel": "attn_fwd_sm100_kernel", "achieved": achieved, "peak": peak,
                     "unit": UNIT, "frac": achieved / peak, "traffic": ATTN_DRAM_TRAFFIC_BYTES,
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this "
                                       "kernel on this workload; a recorded figure, not measured in this run",
                     "ms_per_launch": ms_attn, "peak_source": peak_src},
        "e2e": None if ms_e2e is None else
               {"value": world * flops / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes, "steps": e2e_steps},
        "gpu_launches": 2 * args.steps,
        "clocks": clocks,
    }
    return line


def run_ours(args, rank, world):
    import f2k_cuda_b200 as f2k
    dev = torch.cuda.current_device()
    stream = torch.cuda.current_stream()
    w, p = make_rank_problem(world, rank)
    H = p.q_img.shape[2]
    B, St, Si, D = w.batch, w.seq_txt, w.seq_img, w.head_dim
    flops = 4.0 * B * H * (St + Si) ** 2 * D        # per GPU per step
    tabs = (*f2k.build_rope_4axis_tables((32,) * 4, p.pos_txt, 2000.0),
            *f2k.build_rope_4axis_tables((32,) * 4, p.pos_img, 2000.0))
    ja = f2k.JointAttention(f2k.JointAttention.Config(B, St, Si, H, D))
    if not ja.ok():
        raise RuntimeError(ja.last_error())
    host = [p.q_txt, p.k_txt, p.v_txt, p.q_img, p.k_img, p.v_img]
    d = [dev_bf16(x) for x in host]
    dg = [dev_bf16(g) for g in p.gammas]
    dtab = [torch.from_numpy(t).cuda() for t in tabs]
    o_t, o_i = torch.empty_like(d[0]), torch.empty_like(d[3])
    ws = torch.empty(ja.fused_workspace_size_bytes(), dtype=torch.uint8, device="cuda")

    def step():
        if not ja.forward_fused(*d, dg, dtab, 1e-6, o_t, o_i, ws):
            raise RuntimeError(ja.last_error())

    for _ in range(max(args.warmup, 3)):
        step()
    if ja.device_status() != 0:
        raise RuntimeError("attention kernel reported a device-side error during warm-up")

    sampler = ClockSampler(dev, period_s=0.001) if rank == 0 else None
    if world > 1:
        torch.distributed.barrier()
    ms = time_region(step, args.steps, stream)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())

    # ---- the attention kernel alone (roofline), on the normalised Q/K the prologue left in ws
    bt = (d[0].numel() * 2 + 255) // 256 * 256
    bi = (d[3].numel() * 2 + 255) // 256 * 256
    qn_t = ws[0:bt].view(torch.bfloat16)[: d[0].numel()].view_as(d[0])
    kn_t = ws[bt:2 * bt].view(torch.bfloat16)[: d[0].numel()].view_as(d[0])
    qn_i = ws[2 * bt:2 * bt + bi].view(torch.bfloat16)[: d[3].numel()].view_as(d[3])
    kn_i = ws[2 * bt + bi:2 * bt + 2 * bi].view(torch.bfloat16)[: d[3].numel()].view_as(d[3])

    def attn_only():
        if not ja.forward(qn_t, kn_t, d[2], qn_i, kn_i, d[5], o_t, o_i, None, 0):
            raise RuntimeError(ja.last_error())

    for _ in range(3):
        attn_only()
    ms_attn = time_region(attn_only, args.steps, stream)
    clocks = sampler.stop() if sampler else None      # the two headline regions: fused step, kernel alone

    # ---- the same fused step back to back for seconds: the chip reaches its power state, the
    # clock samples are many, and the figure is set against the sustained cuBLAS peak
    sustained = None
    if world == 1 and not args.skip_sustained:
        sus_steps = int(np.ceil(args.sustained_seconds / (ms * 1e-3)))
        sus_sampler = ClockSampler(dev, period_s=0.02)
        ms_sus = time_region(step, sus_steps, stream)
        sus_clk = sus_sampler.stop()
        speak, ssrc = measured_peak("bf16_tflops_sustained")
        sustained = {"ms_per_step": ms_sus, "steps": sus_steps, "seconds": ms_sus * sus_steps * 1e-3,
                     "value": flops / (ms_sus * 1e-3) / 1e12, "unit": UNIT,
                     "frac_of_sustained_peak": flops / (ms_sus * 1e-3) / 1e12 / speak, "peak": speak, "peak_source": ssrc,
                     "clocks": sus_clk, "clock_bins": sus_sampler.bins(),
                     "ms_x_sm_mhz": None if not sus_clk.get("sm_mhz") else ms_sus * sus_clk["sm_mhz"]}

    # ---- one denoise step of the transformer: 8 double-stream calls (text and image streams
    # separate) + 24 single-stream calls (one combined 4608-token stream), as one CUDA graph
    denoise = denoise_cfg = None
    if world == 1 and not args.skip_denoise_step:
        denoise = denoise_step_leg(d, dg, dtab, o_t, o_i, B, St, Si, H, D, stream, flops, guidance=False)
        denoise_cfg = denoise_step_leg(d, dg, dtab, o_t, o_i, B, St, Si, H, D, stream, flops, guidance=True)

    # ---- end to end through host buffers
    ms_e2e, e2e_steps = None, 0
    hin = [pinned(x) for x in host] if not args.skip_e2e else []
    if not args.skip_e2e:
        ho_t, ho_i = torch.empty_like(hin[0]).pin_memory(), torch.empty_like(hin[3]).pin_memory()

        def step_host():
            if not ja.forward_fused_host(*hin, dg, dtab, 1e-6, ho_t, ho_i):
                raise RuntimeError(ja.last_error())

        for _ in range(3):
            step_host()
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
        e2e_steps = max(3, min(args.steps, 20))
        e2e_sampler = ClockSampler(dev) if rank == 0 else None
        ms_e2e = time_region(step_host, e2e_steps, stream)
        if clocks is not None:
            clocks["e2e_region"] = e2e_sampler.stop()
        if world > 1:
            t = torch.tensor([ms_e2e], device="cuda", dtype=torch.float64)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms_e2e = float(t.item())
    status = ja.device_status()
    if status != 0:
        raise RuntimeError("attention kernel reported a device-side error")

    # ---- N > 1: the fixed jobs of the north star, after the headline legs (whose figures are final
    # by now). A watchdog prints the headline line without them should a job ever stall.
    strong = None
    if world > 1 and not args.skip_strong_scaling:
        hin = None
        torch.cuda.empty_cache()
        result = {}

        def headline_only():
            if rank == 0:
                result["line"]["strong_scaling"] = {"error": "stalled: abandoned after %d s" % STRONG_SECTION_LIMIT_S}
                print(json.dumps(result["line"]), flush=True)
            os._exit(0)

        import threading
        watchdog = threading.Timer(STRONG_SECTION_LIMIT_S, headline_only)
        watchdog.daemon = True
        if rank == 0:
            result["line"] = _headline_line(args, world, flops, ms, ms_attn, ms_e2e, e2e_steps, d, o_t, o_i, clocks, B, H,
                                            St, Si, D)
        watchdog.start()
        try:
            strong = strong_scaling_section(rank, world, only=tuple(x for x in args.strong_jobs.split(",") if x))
        except Exception as exc:
            strong = {"error": f"{type(exc).__name__}: {exc}"}
        watchdog.cancel()
    if rank != 0:
        return None

    line = _headline_line(args, world, flops, ms, ms_attn, ms_e2e, e2e_steps, d, o_t, o_i, clocks, B, H, St, Si, D)
    if strong is not None:
        line["strong_scaling"] = strong
    if sustained is not None:
        line["sustained"] = sustained
    if denoise is not None:
        line["denoise_step"] = denoise
        line["denoise_step_cfg"] = denoise_cfg
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(p, tabs, flops / H)
    if world == 1 and not args.no_reference_kernel:
        # the reference's own kernels, rebuilt for sm_100a, in this same run on this same GPU
        import copy
        a = copy.copy(args)
        a.steps, a.warmup = 5, 3
        try:
            r = run_reference(a, 0, 1)
        except Exception as exc:  # the comparison leg must not take the measurement down with it
            r = {"unavailable": f"{type(exc).__name__}: {exc}"}
        line["reference_kernel"] = (
            {"unavailable": r["unavailable"]} if "unavailable" in r else
            {"value": r["value"], "unit": UNIT, "ms_per_step": r["ms_per_step"], "e2e_value": r["e2e"]["value"],
             "steps": a.steps, "what": r["config"]["step"]})
    return line


# --------------------------------------------------------------------------------------------
# Strong-scaling jobs: a fixed job spread over the GPUs by heads, by sequence (K/V shards pulled by
# the copy engines under the kernel) or by head exchange (sequence outside, heads inside).
# Each set-up returns the step, the figures that describe it, and a parity check of rank 0's
# output against the reference's own kernels (rebuilt for sm_100a) on the same inputs.
# --------------------------------------------------------------------------------------------
SHAPES = {"s4608_b4": "s4608_b4", "s8704": "s8704_edit", "s16896": "s16896"}


def _shape_of(job: str):
    from f2k_cuda_b200.inputs import WORKLOADS
    return WORKLOADS[SHAPES[job.rsplit("_", 1)[0]]]


def _tables(w):
    import f2k_cuda_b200 as f2k
    from f2k_cuda_b200.inputs import token_positions
    pt, pi = token_positions(w)
    return (*f2k.build_rope_4axis_tables((32,) * 4, pt, 2000.0), *f2k.build_rope_4axis_tables((32,) * 4, pi, 2000.0))


def _gains():
    from f2k_cuda_b200.inputs import WORKLOADS, make_problem
    return [dev_bf16(g) for g in make_problem(WORKLOADS["s1152"], heads=1).gammas]


def _device_metrics(got, ref):
    a, b = got.double().flatten(), ref.double().flatten()
    return {"max_abs": float((a - b).abs().max()), "cosine": float((a @ b) / ((a @ a).sqrt() * (b @ b).sqrt())),
            "gate": "max_abs <= 2e-2 and cosine >= 0.9999", "against": "the reference's kernels rebuilt for sm_100a, same inputs"}


def _reference_streams(ref, streams, B, H, D):
    """The reference's block sequence (rmsnorm_bf16, rope_4axis_inplace_bf16, then JointAttention or
    Attention::forward) over one or two streams of raw (q, k, v, gain_q, gain_k, cos, sin)."""
    L = ref.lib
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    prepared = []
    for q, k, v, gq, gk, cos, sin in streams:
        seq = q.shape[1]
        q, k = q.clone(), k.clone()
        rows = B * seq * H
        pos = ((torch.arange(rows, device="cuda") // H) % seq).to(torch.int32)
        for x, g in ((q, gq), (k, gk)):
            if not (L.f2k_ref_rmsnorm_bf16(P(x), P(g), P(x), rows, D, 1e-6, None) and
                    L.f2k_ref_rope_4axis_inplace_bf16(P(x), P(cos), P(sin), P(pos), rows, D, seq, None)):
                raise RuntimeError("reference prologue launch failed")
        prepared.append((q, k, v))
    outs = [torch.empty_like(q) for q, _, _ in prepared]
    if len(prepared) == 2:
        (qt, kt, vt), (qi, ki, vi) = prepared
        h = L.f2k_ref_joint_create(B, qt.shape[1], qi.shape[1], H, D, 0.0)
        n = L.f2k_ref_joint_workspace_bytes(h)
        ws = torch.empty(n, dtype=torch.uint8, device="cuda")
        ok = L.f2k_ref_joint_ok(h) and L.f2k_ref_joint_forward(h, P(qt), P(kt), P(vt), P(qi), P(ki), P(vi), P(outs[0]),
                                                               P(outs[1]), P(ws), n, None)
        torch.cuda.synchronize()
        L.f2k_ref_joint_destroy(h)
    else:
        (q, k, v), = prepared
        h = L.f2k_ref_attn_create(B, q.shape[1], H, D, 0.0)
        ok = L.f2k_ref_attn_ok(h) and L.f2k_ref_attn_forward(h, P(q), P(k), P(v), P(outs[0]), None)
        torch.cuda.synchronize()
        L.f2k_ref_attn_destroy(h)
    if not ok:
        raise RuntimeError("reference attention launch failed")
    return outs


def _gather_tokens(x, world):
    """[1, per, H, D] shards of all ranks -> [1, world * per, H, D] on every rank."""
    if world == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(world)]
    torch.distributed.all_gather(parts, x.contiguous())
    return torch.cat(parts, 1)


def setup_heads(job, rank, world, group_world=None):
    """The job's 32 heads sharded 32/world per GPU: no traffic between the GPUs inside the step.
    Inputs are drawn on the device (N(0,1), seeded per rank); gains and RoPE tables as in the
    headline workload."""
    import f2k_cuda_b200 as f2k
    w = _shape_of(job)
    B, St, Si, D = w.batch, w.seq_txt, w.seq_img, w.head_dim
    H = w.n_heads // world
    dtab = [torch.from_numpy(t).cuda() for t in _tables(w)]
    dg = _gains()
    gen = torch.Generator(device="cuda").manual_seed(4321 + rank)
    mk = lambda n: torch.randn(B, n, H, D, device="cuda", generator=gen).to(torch.bfloat16)  # noqa: E731
    d = [mk(St), mk(St), mk(St), mk(Si), mk(Si), mk(Si)]
    ja = f2k.JointAttention(f2k.JointAttention.Config(B, St, Si, H, D))
    if not ja.ok():
        raise RuntimeError(ja.last_error())
    o_t, o_i = torch.empty_like(d[0]), torch.empty_like(d[3])
    ws = torch.empty(ja.fused_workspace_size_bytes(), dtype=torch.uint8, device="cuda")

    def step():
        if not ja.forward_fused(*d, dg, dtab, 1e-6, o_t, o_i, ws):
            raise RuntimeError(ja.last_error())

    def parity(ref):
        r_t, r_i = _reference_streams(ref, [(d[0], d[1], d[2], dg[0], dg[1], dtab[0], dtab[1]),
                                            (d[3], d[4], d[5], dg[2], dg[3], dtab[2], dtab[3])], B, H, D)
        return _device_metrics(torch.cat([o_t, o_i], 1), torch.cat([r_t, r_i], 1))

    return {"step": step, "status": ja.device_status, "parity": parity, "launches_per_step": 2,
            "flops_total": 4.0 * B * w.n_heads * float(St + Si) ** 2 * D, "nvlink_bytes_per_gpu_per_step": 0,
            "workload": f"{w.name}: {St + Si} tokens, batch {B}, hd128, 32 heads sharded {H} per GPU",
            "step_text": "fused QK-RMSNorm + 4-axis RoPE + non-causal attention, one call",
            "parallelism": f"heads{world}" if world > 1 else "single",
            "l2": "Q, K, V, O and workspace of a step (%.0f MB per GPU) exceed the 126 MB L2"
                  % (6 * B * (St + Si) * H * D * 2 / 1e6)}


def _seq_shard_inputs(w, rank, world):
    """This rank's tokens of the text||image sequence: raw Q, K, V drawn on the device, the rows of
    the combined RoPE tables, and how many of the tokens are text (they come first)."""
    S, H, D = w.seq, w.n_heads, w.head_dim
    if S % world != 0 or H % world != 0:
        raise SystemExit(f"{S} tokens / {H} heads do not split evenly over {world} ranks")
    per = S // world
    b, e = rank * per, (rank + 1) * per
    tabs = _tables(w)
    cos = np.concatenate([tabs[0], tabs[2]])
    sin = np.concatenate([tabs[1], tabs[3]])
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    mk = lambda: torch.randn(1, per, H, D, device="cuda", generator=gen).to(torch.bfloat16)  # noqa: E731
    q_raw, k_raw, v = mk(), mk(), mk()
    return per, b, e, q_raw, k_raw, v, cos, sin, max(0, min(e, w.seq_txt) - b)


def setup_seqpar(job, rank, world, overlap=True):
    """Sequence-parallel attention, batch 1, 32 heads: every rank owns S/world tokens. Step = QK-norm +
    RoPE of the local Q and K, the pulls of the other ranks' K/V shards by the copy engines (readiness
    is exchanged as words in the shard buffers, no collective) and the attention kernel that consumes
    them as they arrive. V is already in the shard buffer (where a V projection would write it)."""
    from f2k_cuda_b200.seqpar import SequenceParallelAttention, qk_norm_rope
    w = _shape_of(job)
    S, H, D = w.seq, w.n_heads, w.head_dim
    per, b, e, q_raw, k_raw, v, cos, sin, n_txt = _seq_shard_inputs(w, rank, world)
    g = _gains()
    dcos, dsin = torch.from_numpy(cos[b:e].copy()).cuda(), torch.from_numpy(sin[b:e].copy()).cuda()
    sp = SequenceParallelAttention(1, per, H, D, world, rank)
    if not sp.ok():
        raise RuntimeError(sp.last_error())
    if not (sp.attach_distributed() if world > 1 else sp.attach_in_process([sp])):
        raise RuntimeError("attaching the peers' shard buffers failed: " + sp.last_error())
    qn, o = torch.empty_like(q_raw), torch.empty_like(q_raw)
    for _ in range(2):                                # V into both buffer sets
        ks, vs = sp.local_kv()
        vs.copy_(v)
        ks.zero_()
        sp.forward(q_raw, o, overlap=False)
    torch.cuda.synchronize()

    def norm_rope(x, y, g_txt, g_img):
        okk = True
        if n_txt > 0:
            okk &= qk_norm_rope(x[:, :n_txt], y[:, :n_txt], g_txt, dcos[:n_txt], dsin[:n_txt], 1e-6)
        if n_txt < per:
            okk &= qk_norm_rope(x[:, n_txt:], y[:, n_txt:], g_img, dcos[n_txt:], dsin[n_txt:], 1e-6)
        return okk

    def step():
        ks, _ = sp.local_kv()
        okk = norm_rope(q_raw, qn, g[0], g[2]) and norm_rope(k_raw, ks, g[1], g[3])
        if not (okk and sp.forward(qn, o, overlap=overlap)):
            raise RuntimeError(sp.last_error())

    def parity(ref):
        qa, ka, va = (_gather_tokens(x, world) for x in (q_raw, k_raw, v))      # collective: every rank calls it
        if rank != 0:
            return None
        dc, ds = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
        t = w.seq_txt
        r_t, r_i = _reference_streams(ref, [(qa[:, :t].contiguous(), ka[:, :t].contiguous(), va[:, :t].contiguous(),
                                             g[0], g[1], dc[:t], ds[:t]),
                                            (qa[:, t:].contiguous(), ka[:, t:].contiguous(), va[:, t:].contiguous(),
                                             g[2], g[3], dc[t:], ds[t:])], 1, H, D)
        return _device_metrics(o, torch.cat([r_t, r_i], 1)[:, b:e])

    return {"step": step, "status": sp.device_status, "parity": parity,
            "launches_per_step": (4 if 0 < n_txt < per else 2) + 1, "flops_total": 4.0 * H * float(S) ** 2 * D,
            "nvlink_bytes_per_gpu_per_step": 2 * (world - 1) * per * H * D * 2,
            "workload": f"{w.name}: {S} tokens, batch 1, 32 heads, hd128, sequence sharded {per} tokens per GPU",
            "step_text": "QK-RMSNorm + RoPE of the local Q, K; copy-engine pulls of the remote K/V shards "
                         + ("under" if overlap else "after which") + " the attention kernel",
            "parallelism": f"seq{world}", "l2": "K/V of all ranks (%.0f MB) exceed the 126 MB L2" % (2 * S * H * D * 2 / 1e6),
            "keep": sp}


def setup_hx(job, rank, world, mode="scatter"):
    """Sequence-parallel attention by head exchange, batch 1, 32 heads: every rank owns S/world tokens
    outside and 32/world heads inside. Step = one kernel that normalises + rotates Q, K and scatters
    Q, K, V by head into the peers' memory, the attention kernel (its epilogue stores each output row
    into the token owner's memory), and the wait for the other ranks' rows. No collective and no
    copy engine in the step. mode "fused": the exchange runs on the attention kernel's spare warps
    (one kernel per step); mode "copy": a prologue kernel, then copy engines deliver the head
    columns under the attention kernel."""
    from f2k_cuda_b200.headswap import HeadExchangeAttention
    w = _shape_of(job)
    S, H, D = w.seq, w.n_heads, w.head_dim
    per, b, e, q_raw, k_raw, v, cos, sin, _ = _seq_shard_inputs(w, rank, world)
    g = _gains()
    dcos, dsin = torch.from_numpy(cos[b:e].copy()).cuda(), torch.from_numpy(sin[b:e].copy()).cuda()
    hx = HeadExchangeAttention(per, H, D, world, rank)
    if not hx.ok():
        raise RuntimeError(hx.last_error())
    if not (hx.attach_distributed() if world > 1 else hx.attach_in_process([hx])):
        raise RuntimeError("attaching the peers' exchange buffers failed: " + hx.last_error())
    if world > 1:
        torch.distributed.barrier()
    out = [None]

    def step():
        # one gain pair for the whole sequence (the single-stream block's call)
        a = (q_raw, k_raw, v, g[2], g[3], dcos, dsin, 1e-6)
        okk = (hx.forward(*a) if mode == "fused" else
               (hx.exchange_in_copy(*a) if mode == "copy" else hx.exchange_in(*a)) and hx.attend())
        if not okk:
            raise RuntimeError(hx.last_error())
        out[0] = hx.output()
        if out[0] is None:
            raise RuntimeError(hx.last_error())

    def parity(ref):
        qa, ka, va = (_gather_tokens(x, world) for x in (q_raw, k_raw, v))
        if rank != 0:
            return None
        dc, ds = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
        (r,) = _reference_streams(ref, [(qa, ka, va, g[2], g[3], dc, ds)], 1, H, D)
        return _device_metrics(out[0], r[:, b:e])

    return {"step": step, "status": hx.device_status, "parity": parity, "launches_per_step": {"fused": 1, "scatter": 2, "copy": 3}[mode],
            "flops_total": 4.0 * H * float(S) ** 2 * D,
            "nvlink_bytes_per_gpu_per_step": 4 * (world - 1) * per * (H // world) * D * 2,
            "workload": f"{w.name}: {S} tokens, batch 1, 32 heads, hd128, {per} tokens per GPU outside, "
                        f"{H // world} heads per GPU inside",
            "step_text": {"fused": "ONE kernel: its spare warps do QK-RMSNorm + RoPE + the head scatter into peer memory "
                                   "while its other warps attend to what has arrived; ",
                          "copy": "QK-RMSNorm + RoPE of all heads (one kernel); copy engines deliver every rank's head "
                                  "columns while the attention kernel runs on what has arrived, local tokens first; ",
                          "scatter": "QK-RMSNorm + RoPE + head scatter into peer memory (one kernel); then attention; "}[mode] +
                         "the epilogue stores each output row into the token owner's memory; wait for the peers' rows",
            "parallelism": f"headswap{world}_" + mode,
            "l2": "Q, K, V, O of a step (%.0f MB per GPU) exceed the 126 MB L2" % (4 * S * (H // world) * D * 2 / 1e6),
            "keep": hx}


def setup_job(job, rank, world, overlap=True):
    kind = job.rsplit("_", 1)[1]
    if kind == "heads":
        return setup_heads(job, rank, world)
    if kind in ("hx", "hxfused", "hxce"):
        return setup_hx(job, rank, world, mode={"hx": "scatter", "hxfused": "fused", "hxce": "copy"}[kind])
    return setup_seqpar(job, rank, world, overlap)


def time_job(j, steps, warmup, rank, world, sample_clocks=True):
    """Warm up, then time `steps` steps between barriers; max over ranks. Returns (ms, clocks)."""
    stream = torch.cuda.current_stream()
    for _ in range(max(warmup, 3)):
        j["step"]()
    if j["status"]() != 0:
        raise RuntimeError("attention kernel reported a device-side error during warm-up")
    sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 and sample_clocks else None
    if world > 1:
        torch.distributed.barrier()
    ms = time_region(j["step"], steps, stream)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop() if sampler else None
    if j["status"]() != 0:
        raise RuntimeError("attention kernel reported a device-side error")
    return ms, clocks


def run_strong(args, rank, world):
    """One strong-scaling job as the whole measurement (--workload <shape>_<heads|seqpar|hx>)."""
    j = setup_job(args.workload, rank, world, overlap=not args.no_overlap)
    ms, clocks = time_job(j, args.steps, args.warmup, rank, world)
    if rank != 0:
        return None
    flops = j["flops_total"]
    peak, peak_src = measured_peak()
    return {
        "metric": METRIC, "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": j["workload"], "step": j["step_text"], "flops_per_step_total": flops,
                   "parallelism": j["parallelism"], "nvlink_bytes_per_gpu_per_step": j["nvlink_bytes_per_gpu_per_step"],
                   "l2": j["l2"]},
        "per_gpu_tflops": flops / world / (ms * 1e-3) / 1e12,
        "pct_of_peak": 100.0 * flops / world / (ms * 1e-3) / 1e12 / peak, "peak_source": peak_src,
        "e2e": None, "gpu_launches": j["launches_per_step"] * args.steps, "clocks": clocks,
    }


STRONG_JOBS = ("s4608_b4_heads", "s16896_heads", "s16896_seqpar", "s16896_hx", "s16896_hxfused", "s16896_hxce", "s8704_heads",
               "s8704_seqpar", "s8704_hx")


def strong_scaling_section(rank, world, min_seconds=0.5, only=()):
    """The fixed jobs the north star names, spread over the `world` GPUs of this run three ways
    (heads, sequence, head exchange), each beside rank 0's own one-GPU time of the same job taken in
    this same run: efficiency = t1 / (world * t_world). Every timed region lasts at least
    `min_seconds`. Parity: rank 0's output rows against the reference's kernels on the gathered
    inputs."""
    import oracle
    ref = oracle.load_ref()
    peak, _ = measured_peak()
    out = {"min_seconds_per_job": min_seconds, "jobs": {}, "one_gpu": {},
           "efficiency": "t1 / (n_gpus * ms_per_step): t1 = rank 0 alone, same job, same run, plain fused call"}

    def n_steps(flops_per_gpu):
        return max(10, int(np.ceil(min_seconds / (flops_per_gpu / 1.0e15))))

    # rank 0 alone: the whole job on one GPU (the other ranks wait at the barrier inside time_job of the next job)
    t1 = {}
    jobs = [j for j in STRONG_JOBS if not only or j in only]
    for shape in ("s4608_b4", "s16896", "s8704"):
        if rank == 0 and any(j.startswith(shape + "_") for j in jobs):
            j = setup_heads(shape + "_heads", 0, 1)
            steps = n_steps(j["flops_total"])
            ms, clocks = time_job(j, steps, 3, 0, 1)
            t1[shape] = ms
            out["one_gpu"][shape] = {"ms_per_step": ms, "steps": steps, "tflops": j["flops_total"] / (ms * 1e-3) / 1e12,
                                     "clocks": clocks}
            del j
            torch.cuda.empty_cache()
    for job in jobs:
        rec = {}
        try:
            j = setup_job(job, rank, world)
            steps = n_steps(j["flops_total"] / world)
            ms, clocks = time_job(j, steps, 3, rank, world)
            par = j["parity"](ref) if ref is not None else None
            if rank == 0:
                shape = job.rsplit("_", 1)[0]
                rec = {"ms_per_step": ms, "steps": steps, "t1_ms": t1[shape], "efficiency": t1[shape] / (world * ms),
                       "tflops_total": j["flops_total"] / (ms * 1e-3) / 1e12,
                       "pct_of_peak_per_gpu": 100.0 * j["flops_total"] / world / (ms * 1e-3) / 1e12 / peak,
                       "nvlink_bytes_per_gpu_per_step": j["nvlink_bytes_per_gpu_per_step"],
                       "nvlink_gb_per_s_per_gpu": j["nvlink_bytes_per_gpu_per_step"] / (ms * 1e-3) / 1e9,
                       "parallelism": j["parallelism"], "workload": j["workload"], "clocks": clocks,
                       "parity": par if par is not None else "oracle/_ref not built"}
            del j
        except Exception as exc:  # one job must not take the others (or the headline) down
            rec = {"error": f"{type(exc).__name__}: {exc}"}
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        if world > 1:
            torch.distributed.barrier()
        if rank == 0:
            out["jobs"][job] = rec
    return out if rank == 0 else None


def run_reference(args, rank, world):
    """The reference's own implementation of the path: its CUDA kernels (rmsnorm_bf16 x4,
    rope_4axis_inplace_bf16 x4, JointAttention::forward with its concat/split copies), rebuilt
    unmodified for sm_100a. It has no CPU implementation and no multi-GPU code: rank 0 runs the
    one-GPU workload, other ranks leave."""
    if rank != 0:
        return None
    import oracle
    ref = oracle.load_ref()
    if ref is None:
        return {"impl": "reference", "unavailable": "oracle/_ref/libf2k_ref.so not built (no reference checkout at build time)"}
    L = ref.lib
    dev = torch.cuda.current_device()
    stream = torch.cuda.current_stream()
    w, p = make_rank_problem(1, 0)
    B, St, Si, H, D = w.batch, w.seq_txt, w.seq_img, w.n_heads, w.head_dim
    flops = 4.0 * B * H * (St + Si) ** 2 * D
    (ct, st) = ref.build_rope_tables((32,) * 4, p.pos_txt, 2000.0)
    (ci, si) = ref.build_rope_tables((32,) * 4, p.pos_img, 2000.0)
    host = [p.q_txt, p.k_txt, p.v_txt, p.q_img, p.k_img, p.v_img]
    src = [dev_bf16(x) for x in host]
    d = [torch.empty_like(x) for x in src]
    dg = [dev_bf16(g) for g in p.gammas]
    dtab = [torch.from_numpy(t).cuda() for t in (ct, st, ci, si)]
    pos_t = ((torch.arange(B * St * H, device="cuda") // H) % St).to(torch.int32)
    pos_i = ((torch.arange(B * Si * H, device="cuda") // H) % Si).to(torch.int32)
    o_t, o_i = torch.empty_like(d[0]), torch.empty_like(d[3])
    h = L.f2k_ref_joint_create(B, St, Si, H, D, 0.0)
    if not L.f2k_ref_joint_ok(h):
        return {"impl": "reference", "unavailable": "reference JointAttention refused the shape"}
    ws_bytes = L.f2k_ref_joint_workspace_bytes(h)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    s_ptr = C.c_void_p(stream.cuda_stream)
    launches = [0]

    def compute():
        ok = 1
        for x, g, (c_, s_), pos, seq in ((d[0], dg[0], dtab[0:2], pos_t, St), (d[1], dg[1], dtab[0:2], pos_t, St),
                                         (d[3], dg[2], dtab[2:4], pos_i, Si), (d[4], dg[3], dtab[2:4], pos_i, Si)):
            rows = B * seq * H
            ok &= L.f2k_ref_rmsnorm_bf16(P(x), P(g), P(x), rows, D, 1e-6, s_ptr)
            ok &= L.f2k_ref_rope_4axis_inplace_bf16(P(x), P(c_), P(s_), P(pos), rows, D, seq, s_ptr)
        ok &= L.f2k_ref_joint_forward(h, P(d[0]), P(d[1]), P(d[2]), P(d[3]), P(d[4]), P(d[5]), P(o_t), P(o_i),
                                      P(ws), ws_bytes, s_ptr)
        launches[0] += 13
        if not ok:
            raise RuntimeError("reference launch failed")

    def step():
        # the reference normalises in place, so each step starts from a fresh copy of the raw q, k
        for dst, s_ in zip(d, src):
            dst.copy_(s_, non_blocking=True)
        compute()

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(dev)
    launches[0] = 0
    ms = time_region(step, args.steps, stream)
    n_launch = launches[0]
    # the device-to-device refresh copies are not part of the reference's path: time them alone and take them out
    ms_copy = time_region(lambda: [dst.copy_(s_, non_blocking=True) for dst, s_ in zip(d, src)], args.steps, stream)
    ms_path = max(ms - ms_copy, 1e-6)

    hin = [pinned(x) for x in host]
    ho_t, ho_i = torch.empty_like(hin[0]).pin_memory(), torch.empty_like(hin[3]).pin_memory()

    def step_host():
        for dst, s_ in zip(d, hin):
            dst.copy_(s_, non_blocking=True)
        compute()
        ho_t.copy_(o_t, non_blocking=True)
        ho_i.copy_(o_i, non_blocking=True)

    for _ in range(2):
        step_host()
    e2e_steps = max(3, min(args.steps, 20))
    ms_e2e = time_region(step_host, e2e_steps, stream)
    clocks = sampler.stop()
    L.f2k_ref_joint_destroy(h)
    peak, peak_src = measured_peak()
    val = flops / (ms_path * 1e-3) / 1e12
    return {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_path, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": HEADLINE_WORKLOAD,
                   "step": "reference kernels rebuilt for sm_100a: rmsnorm_bf16 x4, rope_4axis_inplace_bf16 x4, "
                           "JointAttention::forward (3 concat + flash_mma_kernel<128> + split)",
                   "flops_per_step_per_gpu": flops, "ranks_used": 1,
                   "note": "the reference's implementation of this path is CUDA only (no CPU code, no multi-GPU code)"},
        "pct_of_peak": 100.0 * val / peak, "peak_source": peak_src,
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": 0, "kind": "reference",
                         "sample": "not a CPU run: the reference has no CPU implementation of this path; its own CUDA "
                                   "kernels, rebuilt for sm_100a, on one GPU, full workload"},
        "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": sum(x.numel() * 2 for x in hin),
                "d2h_bytes_per_step": ho_t.numel() * 2 + ho_i.numel() * 2, "steps": e2e_steps},
        "gpu_launches": n_launch, "clocks": clocks,
    }


def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nnodes=1 "
                         "--nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...")
    if 32 % world != 0:
        raise SystemExit("the 32 heads shard over 1, 2, 4, 8, 16 or 32 GPUs")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: the library has no CPU path")
    torch.cuda.set_device(local)
    if args.impl == "reference" and rank != 0:
        return
    if world > 1 and args.impl == "ours":
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
    try:
        if args.impl == "reference":
            line = run_reference(args, rank, world)
        elif args.workload == "s4608":
            line = run_ours(args, rank, world)
        else:
            line = run_strong(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
    finally:
        if world > 1 and args.impl == "ours" and torch.distributed.is_initialized():
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
