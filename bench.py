#!/usr/bin/env python
"""Benchmark of the Mimi attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (benchmark config 3, "batched prefill"): per GPU 512 clips of 250 frames (10 s at 25 Hz)
through the attention path of 16 transformer layers (8 encoder + 8 decoder): QKV projection + RoPE +
banded causal attention (window 250), BF16 inputs, FP32 accumulate.  One step = one pass of the 16
layers over the batch.  Metric: attention frames/s = clips * frames * layers / time, summed over GPUs.
Clips are independent, so ranks share nothing on the data path (weak scaling: 512 clips per GPU).

One JSON line is printed by rank 0.  `value` is device-resident throughput; `e2e` includes the
host->device copy of the batch from pinned memory and the device->host copy of the last layer's output
every step.  `roofline` describes the kernel with the largest share of the step, timed with CUDA events
on the launching stream inside the timed region; `kernels` lists both kernels of the step and, timed after
it, the fused one-kernel form of the same layer call.  `parity` compares the timed configuration's own
output (full-size launches, 8 clips x 16 layers) with the CPU oracle.  `strong` is the same workload with
the 512 clips split over the GPUs (benchmark config 3 as stated), `longclip` benchmark config 4 with its 16
clips split over the GPUs, `host_copy` the pinned-memory copies of the e2e loop without kernels (the
ceiling the host side puts on `e2e`), `decode` the streaming single-frame step (benchmark config 5) on a
full 250-slot ring.  `cpu_baseline` is the CPU arm on a fixed 64-clip sample of the same workload.

`--impl reference` times the CPU arm alone: the reference's own MimiAttention.forward (FP32, all host
threads) where its package has been placed under oracle/_ref by oracle/make_ref.py, else the oracle's
restatement of the same calls; the line's cpu_baseline.kind says which.
`--workload longclip | stream | streamlayer | stack | rvq` print one line each for the secondary workloads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CLIPS, FRAMES, LAYERS, HIDDEN, WINDOW = 512, 250, 16, 512, 250
QKV_FLOP_PER_FRAME = 2 * 512 * 1536
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of each kernel.  ncu cannot run inside this
# script, so these come from the captures summarised under profiles/ (same kernels, a 256-clip case: traffic grows in
# proportion to the clips) scaled by 2 to this workload's 512 clips; the line says so in `traffic_source`.
NCU_TRAFFIC_BYTES_256_CLIPS = {"qkv_rope_gemm_kernel": 217.1e6, "band_attn_clip_kernel": 236.7e6,
                               "attn_fused_clip_kernel": 88.9e6}
DTYPE = "bf16 x, W, q, k / fp16 v, p, out / fp32 accumulate"


def pairs(t: int, window: int = WINDOW) -> int:
    return sum(min(i + 1, window) for i in range(t))


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Streams SM clocks and throttle reasons from one `nvidia-smi -lms 50` child while the timed
    region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.samples: list[list[str]] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            time.sleep(0.6)      # let the first sample land before the timed region starts
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        for line in out.splitlines():
            cols = [c.strip() for c in line.split(",")]
            if len(cols) == 7:
                self.samples.append(cols)

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        power = [float(s[2]) for s in self.samples if s[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[3 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(self.samples[0][1]),
                "reasons": reasons, "samples": len(self.samples), "power_w_max": max(power) if power else None}


# --------------------------------------------------------------------------- CPU arm
CPU_SAMPLE_CLIPS = 64      # clips per CPU step: the same sample at every --gpus value


def cpu_reference_step(sample_clips: int, layers: int, seed: int = 1):
    """One pass of the attention path over `sample_clips` clips x `layers` layers on the host cores, and which
    code runs it.  Where the reference's package is present (oracle/_ref, placed by oracle/make_ref.py) this is
    the reference's OWN MimiAttention.forward (src/fast_mimi/model.py:1870-1961), FP32, sdpa backend, with its
    rotary tables and the band mask its transformer builds once per stack call (src/fast_mimi/model.py:2192-2206);
    o_proj, which is not part of the timed path of either arm, is replaced by an identity.  Otherwise the oracle's
    restatement of the same calls."""
    import oracle
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(sample_clips, FRAMES, HIDDEN, generator=g)
    ws = [(torch.randn(1536, HIDDEN, generator=g) * 0.02) for _ in range(layers)]
    if oracle.import_reference() is not None:
        from fast_mimi import MimiConfig
        from fast_mimi.model import MimiAttention, MimiRotaryEmbedding, _attention_mask
        cfg = MimiConfig()
        attns = []
        for l, w in enumerate(ws):
            attn = MimiAttention(cfg, l, "sdpa").eval()
            with torch.no_grad():
                for lin, part in zip((attn.q_proj, attn.k_proj, attn.v_proj), w.chunk(3, 0)):
                    lin.weight.copy_(part)
            attn.o_proj = torch.nn.Identity()
            attns.append(attn)
        rope = MimiRotaryEmbedding(cfg)

        def run():
            with torch.inference_mode():
                pe = rope(x, torch.arange(FRAMES)[None])
                mask = _attention_mask(batch_size=sample_clips, query_length=FRAMES, key_length=FRAMES, query_offset=0,
                                       key_offset=0, sliding_window=cfg.sliding_window, padding_mask=None,
                                       backend="sdpa", dtype=x.dtype, device=x.device)
                out = None
                for attn in attns:
                    out, _ = attn(x, mask, None, pe)
                return out

        return run, "reference"

    from oracle import mimi_attention_oracle as O
    cos, sin = O.rope_tables(torch.arange(FRAMES))

    def run_port():
        out = None
        for w in ws:
            q, k, v = O.qkv_project(x, *w.chunk(3, 0))
            q, k = O.apply_rope(q, k, cos, sin)
            out = O.band_attention_sdpa(q, k, v)
        return out

    return run_port, "port"


def time_cpu_baseline(budget_s: float = 12.0) -> dict:
    torch.set_num_threads(os.cpu_count() or 1)
    run, kind = cpu_reference_step(CPU_SAMPLE_CLIPS, LAYERS)
    run()
    reps, t0 = 0, time.perf_counter()
    while reps < 16 and (reps == 0 or time.perf_counter() - t0 < budget_s):
        run()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": CPU_SAMPLE_CLIPS * FRAMES * LAYERS / dt, "unit": "frames/s", "cores": torch.get_num_threads(),
            "kind": kind, "sample": f"{CPU_SAMPLE_CLIPS} of {CLIPS} clips x {FRAMES} frames x {LAYERS} layers, FP32, "
                                    f"mean of {reps} repetitions of {dt:.2f} s after one warm-up"}


def run_reference(args) -> None:
    """The reference's CPU path on the host cores, same metric and config; every step is the same 64-clip sample
    whatever --gpus says, so the lines of a scaling run are comparable."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    clips = CPU_SAMPLE_CLIPS
    run, kind = cpu_reference_step(clips, LAYERS)
    for _ in range(args.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    elapsed = time.perf_counter() - t0
    ms = elapsed / args.steps * 1e3
    value = clips * FRAMES * LAYERS / (ms / 1e3)
    cpu = {"value": value, "unit": "frames/s", "cores": torch.get_num_threads(), "kind": kind,
           "sample": f"each step = {clips} of {CLIPS} clips x {FRAMES} frames x {LAYERS} layers, FP32"
                     + (", the reference's own MimiAttention.forward (o_proj excluded)" if kind == "reference"
                        else ", the oracle's restatement (reference package absent)")}
    print(json.dumps({
        "impl": "reference", "metric": "attention frames/s", "value": value, "unit": "frames/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(), "cpu_baseline": cpu,
        "e2e": {"value": value, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def config_dict() -> dict:
    return {"workload": "batched prefill (benchmark config 3): QKV projection + RoPE + banded causal attention, "
                        "16 layers", "clips_per_gpu": CLIPS, "frames": FRAMES, "layers": LAYERS, "window": WINDOW,
            "heads": 8, "head_dim": 64,
            "l2": "inputs larger than L2: x and out of one layer call are 262 MB, and all 16 calls of a step read the "
                  "same x with different weights and write the same out",
            "kernel": "one launch per layer call: projection + RoPE + banded attention (q, k, v never in memory)"}


# --------------------------------------------------------------------------- GPU arm
def pin_to_gpu_numa_node(gpu_index: int) -> None:
    """Multi-rank runs: keep this rank's threads (and with them the pinned host buffers it allocates next) on
    the CPU cores of the NUMA node its GPU hangs off, so that eight ranks' host<->device copies do not all
    cross the socket interconnect.  Best effort: silently does nothing where sysfs or the call is unavailable."""
    try:
        bus = torch.cuda.get_device_properties(gpu_index).pci_bus_id
        domain = torch.cuda.get_device_properties(gpu_index).pci_domain_id
        dev_id = torch.cuda.get_device_properties(gpu_index).pci_device_id
        path = f"/sys/bus/pci/devices/{domain:04x}:{bus:02x}:{dev_id:02x}.0/local_cpulist"
        cpus: set = set()
        for part in open(path).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            print(f"rank on GPU {gpu_index}: pinned to {len(allowed)} CPUs of its NUMA node", file=sys.stderr)
    except Exception as exc:      # noqa: BLE001 - placement is an optimisation only
        print(f"rank on GPU {gpu_index}: NUMA pinning skipped ({exc})", file=sys.stderr)


def run_ours(args) -> None:
    import torch.distributed as dist
    import fast_mimi_b200 as fm
    from fast_mimi_b200 import ops, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    real_stdout = None
    if world > 1:
        # Libraries write banners to file descriptor 1 (NCCL prints its version there).  Everything but the
        # result line goes to stderr: descriptor 1 is pointed at stderr for the run and the JSON line is written
        # to a saved copy of the real stdout at the end.
        sys.stdout.flush()
        real_stdout = os.dup(1)
        os.dup2(2, 1)
        pin_to_gpu_numa_node(local_rank)
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    g = torch.Generator(device=dev).manual_seed(1 + rank)
    x = torch.randn(CLIPS, FRAMES, HIDDEN, device=dev, generator=g).bfloat16()
    ws = [(torch.randn(1536, HIDDEN, device=dev, generator=g) * 0.02).bfloat16() for _ in range(LAYERS)]
    pos = torch.arange(FRAMES, device=dev, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2, device=dev, dtype=torch.int64).float() / 64))
    freqs = torch.outer(pos, inv)
    emb = torch.cat((freqs, freqs), -1)
    cos, sin = emb.cos()[None].contiguous(), emb.sin()[None].contiguous()
    q = torch.empty_like(x); k = torch.empty_like(x)
    v = torch.empty(x.shape, dtype=torch.float16, device=dev)
    out = torch.empty(x.shape, dtype=torch.float16, device=dev)
    status = ops.new_status(dev)
    stream = torch.cuda.current_stream()

    def step(events=None, xin=None, outbuf=None, clips=CLIPS):
        """One pass of the 16 layers through the public entry point for a cache-free call, ops.attention_prefill
        (for 250-frame clips: one kernel per layer call, projection + RoPE + banded attention)."""
        xin = x if xin is None else xin
        outbuf = out if outbuf is None else outbuf
        for l in range(LAYERS):
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True); e0.record(stream)
            ops.attention_prefill(xin[:clips], ws[l], cos, sin, window=WINDOW, scale=0.125, out=outbuf[:clips], status=status)
            if events is not None:
                e1 = torch.cuda.Event(enable_timing=True); e1.record(stream)
                events.append((e0, e1))

    # ---- device-resident throughput ---------------------------------------------------------
    for _ in range(args.warmup):
        step()
    barrier()
    events: list = []
    start = torch.cuda.Event(enable_timing=True); stop = torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        start.record(stream)
        for _ in range(args.steps):
            step(events)
        stop.record(stream)
        barrier()
    ms_total = start.elapsed_time(stop)
    ops.check_status(status=status)
    fused_ms = statistics.mean(a.elapsed_time(b) for a, b in events)

    # ---- parity of the timed configuration's own output -------------------------------------
    # The buffers of the timed run, full-size launches: every layer's result for the first clips against the CPU
    # oracle on the same values (relative L2, tolerance 2e-3 as in tests/).
    parity = None
    if rank == 0 and not args.no_cpu:
        from oracle import mimi_attention_oracle as O
        n_par = 8
        xs_cpu = x[:n_par].float().cpu()
        cos_c, sin_c = O.rope_tables(torch.arange(FRAMES))
        worst = 0.0
        worst_two = 0.0
        out_2 = torch.empty_like(out)
        for l in range(LAYERS):
            ops.attention_prefill(x, ws[l], cos, sin, window=WINDOW, scale=0.125, out=out, status=status)
            ops.qkv_rope(x, ws[l], cos, sin, out=(q, k, v), status=status)
            ops.band_attention_prefill(q, k, v, window=WINDOW, scale=0.125, out=out_2, status=status)
            got = out[:n_par].float().cpu()
            qc, kc, vc = O.qkv_project(xs_cpu, *ws[l].float().cpu().chunk(3, 0))
            qc, kc = O.apply_rope(qc, kc, cos_c, sin_c)
            want = O.band_attention(qc, kc, vc).transpose(1, 2).reshape(n_par, FRAMES, HIDDEN)
            worst = max(worst, O.rel_l2(got, want))
            worst_two = max(worst_two, O.rel_l2(out_2[:n_par].float().cpu(), want))
        del out_2
        parity = {"rel_l2_max": worst, "clips": n_par, "layers": LAYERS, "tolerance": 2e-3, "ok": worst <= 2e-3,
                  "rel_l2_max_two_kernel_form": worst_two,
                  "what": "output of the full-size launches of the timed configuration vs the CPU oracle"}

    # ---- the same layer call as two kernels (projection + RoPE, then attention, q / k / v through HBM); not in the step ----
    two_events: list = []
    for it in range(3 + 8):
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True); e2 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        ops.qkv_rope(x, ws[it % LAYERS], cos, sin, out=(q, k, v), status=status)
        e1.record(stream)
        ops.band_attention_prefill(q, k, v, window=WINDOW, scale=0.125, out=out, status=status)
        e2.record(stream)
        if it >= 3:
            two_events.append((e0, e1, e2))
    torch.cuda.synchronize()
    gemm_ms = statistics.mean(a.elapsed_time(b) for a, b, _ in two_events)
    attn_ms = statistics.mean(b.elapsed_time(c) for _, b, c in two_events)

    # ---- end to end: pinned host input -> device -> 16 layers -> host --------------------------
    # Every step copies its batch in from pinned memory and its result out; the copies of neighbouring
    # steps run on their own streams (two device buffers each way), so a step's transfer overlaps the
    # previous step's kernels, as a serving loop would do it.
    x_host = torch.empty(x.shape, dtype=x.dtype, pin_memory=True); x_host.copy_(x)
    out_hosts = [torch.empty(out.shape, dtype=out.dtype, pin_memory=True) for _ in range(2)]
    x_devs = [x, torch.empty_like(x)]
    out_devs = [out, torch.empty_like(out)]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def e2e_run(n_steps, compute=True):
        in_ready = [None, None]; computed = [None, None]; copied_out = [None, None]
        for i in range(n_steps):
            b = i & 1
            with torch.cuda.stream(s_in):
                if computed[b] is not None:
                    s_in.wait_event(computed[b])            # x_devs[b] is free once step i-2 has consumed it
                x_devs[b].copy_(x_host, non_blocking=True)
                in_ready[b] = torch.cuda.Event(); in_ready[b].record(s_in)
            stream.wait_event(in_ready[b])
            if copied_out[b] is not None:
                stream.wait_event(copied_out[b])            # out_devs[b] has left for the host
            if compute:
                step(xin=x_devs[b], outbuf=out_devs[b])
            computed[b] = torch.cuda.Event(); computed[b].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed[b])
                out_hosts[b].copy_(out_devs[b], non_blocking=True)
                copied_out[b] = torch.cuda.Event(); copied_out[b].record(s_out)
        for ev in copied_out:
            if ev is not None:
                stream.wait_event(ev)

    e2e_run(max(2, args.warmup // 2))
    barrier()
    s2 = torch.cuda.Event(enable_timing=True); t2 = torch.cuda.Event(enable_timing=True)
    s2.record(stream)
    e2e_run(args.steps)
    t2.record(stream)
    barrier()
    ms_e2e = s2.elapsed_time(t2)
    # The same loop without the kernels: what the host side alone can carry (all ranks at once).
    e2e_run(2, compute=False)
    barrier()
    s3 = torch.cuda.Event(enable_timing=True); t3 = torch.cuda.Event(enable_timing=True)
    s3.record(stream)
    e2e_run(10, compute=False)
    t3.record(stream)
    barrier()
    ms_copy = s3.elapsed_time(t3) / 10

    # ---- strong scaling: the batch of benchmark config 3 (512 clips in total) split over the ranks -----------
    lo, hi = sharding.shard_bounds(CLIPS, world, rank)
    n_strong = hi - lo
    for _ in range(3):
        step(clips=n_strong)
    barrier()
    s4 = torch.cuda.Event(enable_timing=True); t4 = torch.cuda.Event(enable_timing=True)
    s4.record(stream)
    for _ in range(args.steps):
        step(clips=n_strong)
    t4.record(stream)
    barrier()
    ms_strong = s4.elapsed_time(t4) / args.steps

    # ---- long clips (benchmark config 4): 16 clips of 2500 frames split over the ranks ------------------------
    longclip = bench_longclip(dev, stream, peaks, world, rank)

    # ---- streaming decode (benchmark config 5) on a full ring ----------------------------------
    decode = None
    if not args.no_decode:
        decode = bench_decode(dev, stream, peaks, world, rank)

    # ---- the output projection that follows the path (not part of the timed step) -------------
    # y = x + layer_scale * (attn W_o^T) over one layer's frames, on the same GEMM kernel.
    w_o = (torch.randn(HIDDEN, HIDDEN, device=dev, generator=g) * 0.04).half()
    scale_o = torch.full((HIDDEN,), 0.01, device=dev)
    resid = torch.randn(out.shape, device=dev, generator=g).half()
    y = torch.empty_like(out)
    for _ in range(3):
        ops.out_proj(out, w_o, layer_scale=scale_o, residual=resid, out=y, status=status)
    o0 = torch.cuda.Event(enable_timing=True); o1 = torch.cuda.Event(enable_timing=True)
    o0.record(stream)
    for _ in range(10):
        ops.out_proj(out, w_o, layer_scale=scale_o, residual=resid, out=y, status=status)
    o1.record(stream)
    torch.cuda.synchronize()
    ops.check_status(status=status)
    oproj_ms = o0.elapsed_time(o1) / 10
    oproj_bytes = 3 * out.numel() * 2
    out_proj = {"kernel": "qkv_rope_gemm_kernel (output projection + layer scale + residual)", "ms": oproj_ms,
                "tflops": out.shape[0] * out.shape[1] * 2 * HIDDEN * HIDDEN / (oproj_ms / 1e3) / 1e12,
                "gbs": oproj_bytes / (oproj_ms / 1e3) / 1e9, "frac_hbm": oproj_bytes / (oproj_ms / 1e3) / 1e9 / peaks["hbm_gbs"],
                "note": "next step after the timed path; not included in value or e2e"}

    times = torch.tensor([ms_total, ms_e2e, fused_ms, gemm_ms, attn_ms, ms_copy, ms_strong], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e, fused_ms, gemm_ms, attn_ms, ms_copy, ms_strong = times.tolist()
    frames_per_step = CLIPS * FRAMES * LAYERS * world
    ms_per_step = ms_total / args.steps
    value = frames_per_step / (ms_per_step / 1e3)
    e2e_value = frames_per_step / (ms_e2e / args.steps / 1e3)

    rows = CLIPS * FRAMES
    gemm_flop = rows * QKV_FLOP_PER_FRAME
    attn_flop = CLIPS * 2048 * pairs(FRAMES)
    attn_bytes = 4 * rows * HIDDEN * 2
    fused_bytes = 2 * rows * HIDDEN * 2
    fused_tf = (gemm_flop + attn_flop) / (fused_ms / 1e3) / 1e12
    gemm_tf = gemm_flop / (gemm_ms / 1e3) / 1e12
    attn_gbs = attn_bytes / (attn_ms / 1e3) / 1e9

    def traffic(name):
        t = NCU_TRAFFIC_BYTES_256_CLIPS.get(name)
        return None if t is None else 2 * t

    kernels = [
        {"kernel": "attn_fused_clip_kernel", "in_step": True, "ms": fused_ms, "share": 1.0, "bound": "tensor",
         "achieved": fused_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": fused_tf / peaks["bf16_tflops"],
         "frac_sustained": fused_tf / peaks["bf16_tflops_sustained"],
         "gbs": fused_bytes / (fused_ms / 1e3) / 1e9, "algorithmic_flop": gemm_flop + attn_flop, "algorithmic_bytes": fused_bytes,
         "note": "the whole layer call in one kernel: x in, attention out (893 FLOP per HBM byte: tensor-bound)"},
        {"kernel": "qkv_rope_gemm_kernel", "in_step": False, "ms": gemm_ms,
         "bound": "tensor", "achieved": gemm_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
         "frac": gemm_tf / peaks["bf16_tflops"], "frac_sustained": gemm_tf / peaks["bf16_tflops_sustained"],
         "algorithmic_flop": gemm_flop,
         "note": "first half of the two-kernel form of the same call (other clip lengths, cached calls); timed after the step"},
        {"kernel": "band_attn_clip_kernel", "in_step": False, "ms": attn_ms,
         "bound": "hbm", "achieved": attn_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": attn_gbs / peaks["hbm_gbs"],
         "frac_sustained": attn_gbs / peaks["hbm_gbs"], "tensor_tflops": attn_flop / (attn_ms / 1e3) / 1e12,
         "algorithmic_bytes": attn_bytes,
         "note": "second half of the two-kernel form; timed after the step"},
    ]
    top = kernels[0]
    roofline = {"bound": top["bound"], "achieved": top["achieved"], "peak": top["peak"], "unit": top["unit"],
                "frac": top["frac"], "frac_sustained": top["frac_sustained"], "traffic": traffic(top["kernel"]),
                "traffic_source": "profiles/ (ncu capture of a 256-clip launch, scaled x2 by the clips processed)",
                "kernel": top["kernel"], "peak_source": f"{peaks['source']} (burst figure; frac_sustained uses the sustained one)",
                "avg_launch_ms": top["ms"]}

    if rank == 0:
        cpu = time_cpu_baseline() if world == 1 and not args.no_cpu else None
        h2d, d2h = x.numel() * 2, out.numel() * 2
        line = {
            "metric": "attention frames/s", "value": value, "unit": "frames/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic", "config": config_dict(),
            "e2e": {"value": e2e_value, "unit": "frames/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": args.steps * LAYERS, "roofline": roofline, "kernels": kernels, "parity": parity,
            "host_copy": {"ms_per_step": ms_copy, "gbs_per_gpu": (h2d + d2h) / (ms_copy / 1e3) / 1e9,
                          "gbs_all_gpus": world * (h2d + d2h) / (ms_copy / 1e3) / 1e9,
                          "what": "the e2e loop's pinned-host copies alone (no kernels), all ranks at once, max over ranks: "
                                  "the ceiling the host side puts on e2e"},
            "strong": {"scaling": "strong", "clips_total": CLIPS, "clips_per_gpu": n_strong, "ms_per_step": ms_strong,
                       "value": CLIPS * FRAMES * LAYERS / (ms_strong / 1e3), "unit": "frames/s",
                       "what": "benchmark config 3 as stated: 512 clips in total, split evenly over the GPUs"},
            "longclip": longclip,
            "clocks": clocks.summary(), "cpu_baseline": cpu, "decode": decode, "out_proj": out_proj,
            "step_tflops": (gemm_flop + attn_flop) * LAYERS / (ms_per_step / 1e3) / 1e12,
        }
        if real_stdout is None:
            print(json.dumps(line))
        else:
            sys.stdout.flush()
            os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def bench_longclip(dev, stream, peaks, world, rank, clips_total: int = 16, T: int = 2500, steps: int = 20) -> dict:
    """Benchmark config 4 (banded attention alone on 16 clips of 2500 frames, rotated BF16 q, k / FP16 v resident),
    the clips split evenly over the ranks; three input sets in rotation so that none survives in L2."""
    import torch.distributed as dist
    from fast_mimi_b200 import ops, sharding
    lo, hi = sharding.shard_bounds(clips_total, world, rank)
    B = hi - lo
    g = torch.Generator(device=dev).manual_seed(11 + rank)
    n_sets = 3 if world == 1 else 3 * world       # per-rank inputs shrink with the split: keep the rotation above L2
    sets = []
    for _ in range(n_sets):
        sets.append(((torch.randn(B, T, 512, device=dev, generator=g) / 8).bfloat16(),
                     (torch.randn(B, T, 512, device=dev, generator=g) / 8).bfloat16(),
                     (torch.randn(B, T, 512, device=dev, generator=g) / 8).half()))
    out = torch.empty_like(sets[0][2])
    for i in range(3):
        ops.band_attention_prefill(*sets[i % n_sets], window=WINDOW, out=out)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for i in range(steps):
        ops.band_attention_prefill(*sets[i % n_sets], window=WINDOW, out=out)
    b.record(stream)
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    nbytes = 4 * clips_total * T * 512 * 2
    gbs = nbytes / (ms / 1e3) / 1e9
    del sets
    torch.cuda.empty_cache()
    return {"workload": "long-clip banded attention (benchmark config 4), one layer call", "clips_total": clips_total,
            "clips_per_gpu": B, "frames": T, "ms_per_call": ms, "value": clips_total * T / (ms / 1e3), "unit": "frames/s",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"] * world, "unit": "GB/s",
                         "frac": gbs / (peaks["hbm_gbs"] * world), "kernel": "band_attn_long_kernel",
                         "tensor_tflops": clips_total * 2048 * pairs(T) / (ms / 1e3) / 1e12}}


def bench_decode(dev, stream, peaks, world, rank, streams: int = 4096, layers: int = 8, steps: int = 20) -> dict:
    """Full-ring streaming steps: 4096 streams x 8 layers, ring position >= 250 (every slot valid)."""
    import torch.distributed as dist
    import fast_mimi_b200 as fm
    from fast_mimi_b200 import ops
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    ring = fm.MimiKVRing(layers, streams, WINDOW, device=dev)
    ring.ring_k.copy_((torch.randn(ring.ring_k.shape[1:], device=dev, generator=g) / 2).bfloat16().expand_as(ring.ring_k))
    ring.ring_v.copy_((torch.randn(ring.ring_v.shape[1:], device=dev, generator=g) / 2).half().expand_as(ring.ring_v))
    ws = [(torch.randn(1536, HIDDEN, device=dev, generator=g) * 0.02).bfloat16() for _ in range(layers)]
    xs = torch.randn(streams, HIDDEN, device=dev, generator=g).bfloat16()
    cos = torch.ones(1, 1, 64, device=dev); sin = torch.zeros(1, 1, 64, device=dev)
    qws = torch.empty_like(xs)
    out = torch.empty(streams, HIDDEN, device=dev, dtype=torch.float32)
    status = ops.new_status(dev)

    def one_step(pos, events=None):
        for l in range(layers):
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True); e0.record(stream)
            ops.decode_step(xs, ws[l], cos, sin, ring.ring_k[l], ring.ring_v[l], pos, q_workspace=qws, out=out,
                            status=status)
            if events is not None:
                e1 = torch.cuda.Event(enable_timing=True); e1.record(stream)
                events.append((e0, e1))

    for i in range(3):
        one_step(250 + i)
    torch.cuda.synchronize()
    events: list = []
    a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for i in range(steps):
        one_step(253 + i, events)
    b.record(stream)
    torch.cuda.synchronize()
    if ops.read_status(status) != 0:
        raise SystemExit("decode: a bounded device wait timed out")
    ms = torch.tensor([a.elapsed_time(b) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms)
    layer_ms = statistics.mean(x.elapsed_time(y) for x, y in events)
    # algorithmic bytes per (stream, layer, step): ring read 2*250*512*2, ring write 2048, x 1024 (bf16), out 2048
    per_stream = 2 * WINDOW * 512 * 2 + 2048 + 1024 + 2048
    bytes_layer = streams * per_stream + 1536 * 512 * 2
    gbs = bytes_layer / (layer_ms / 1e3) / 1e9
    del ring
    torch.cuda.empty_cache()
    return {"workload": "streaming decode (benchmark config 5), full 250-slot ring", "streams_per_gpu": streams,
            "layers": layers, "steps": steps, "ms_per_step": ms_step,
            "value": streams * layers * world / (ms_step / 1e3), "unit": "frames/s",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "kernel": "qkv_rope_gemm_kernel + ring_decode_attn_kernel",
                         "avg_layer_ms": layer_ms, "bytes_per_layer_step": bytes_layer}}


def profile_case(which: str) -> None:
    """Small cases for `ncu --set full` captures (inputs above the 126 MB L2, well under a few GB,
    a handful of launches): prefill = 256 clips x 250 frames, one layer; decode = 512 streams on a
    full ring, one layer; layer = one whole transformer layer on 256 clips x 250 frames (LayerNorm and the
    three epilogue variants of the linear kernel); longclip = 16 clips x 2500 frames, three input sets in
    rotation; rvq = 64 000 vectors through two quantiser layers.  Prints nothing that is a benchmark value."""
    import fast_mimi_b200 as fm
    from fast_mimi_b200 import ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    w = (torch.randn(1536, HIDDEN, device=dev, generator=g) * 0.02).bfloat16()
    if which == "prefill":
        x = torch.randn(256, FRAMES, HIDDEN, device=dev, generator=g).bfloat16()
        cos = torch.ones(1, FRAMES, 64, device=dev); sin = torch.zeros(1, FRAMES, 64, device=dev)
        # the two-kernel form of the call (projection + RoPE, then whole-clip attention), q / k / v through HBM
        qkv = (torch.empty_like(x), torch.empty_like(x), torch.empty(x.shape, dtype=torch.float16, device=dev))
        for _ in range(4):
            ops.qkv_rope(x, w, cos, sin, out=qkv)
            ops.band_attention_prefill(*qkv, window=WINDOW)
    elif which == "fused":
        x = torch.randn(256, FRAMES, HIDDEN, device=dev, generator=g).bfloat16()
        cos = torch.ones(1, FRAMES, 64, device=dev); sin = torch.zeros(1, FRAMES, 64, device=dev)
        for _ in range(4):
            ops.attention_fused(x, w, cos, sin)
    elif which == "chunk":
        # 512 streams, 64 new frames on top of full rings: the offset-key attention kernel and the two ring copies
        ring = fm.MimiKVRing(1, 512, WINDOW, device=dev)
        ring.ring_k.copy_((torch.randn(ring.ring_k.shape, device=dev, generator=g) / 2).bfloat16())
        ring.ring_v.copy_((torch.randn(ring.ring_v.shape, device=dev, generator=g) / 2).half())
        xs = torch.randn(512, 64, HIDDEN, device=dev, generator=g).bfloat16()
        cos = torch.ones(1, 64, 64, device=dev); sin = torch.zeros(1, 64, 64, device=dev)
        for i in range(3):
            ops.attention_chunk(xs, w, cos, sin, ring.ring_k[0], ring.ring_v[0], 300 + 64 * i)
    elif which == "layer":
        layer = fm.MimiTransformerLayerB200().to(dev)
        x = torch.randn(256, FRAMES, HIDDEN, device=dev, generator=g)
        cos = torch.ones(1, FRAMES, 64, device=dev); sin = torch.zeros(1, FRAMES, 64, device=dev)
        with torch.no_grad():
            for _ in range(3):
                layer(x, None, None, (cos, sin), False)
    elif which == "rvq":
        books = ops.RVQCodebooks(torch.randn(2, 2048, 256, device=dev, generator=g))
        xq = torch.randn(64000, 256, device=dev, generator=g) * 1.5
        for _ in range(2):
            ops.rvq_encode(xq, books)
    elif which == "longclip":
        sets = [tuple((torch.randn(16, 2500, HIDDEN, device=dev, generator=g) / 8).to(dt)
                      for dt in (torch.bfloat16, torch.bfloat16, torch.float16)) for _ in range(3)]
        for i in range(4):
            ops.band_attention_prefill(*sets[i % 3], window=WINDOW)
    else:
        ring = fm.MimiKVRing(1, 512, WINDOW, device=dev)
        ring.ring_k.copy_((torch.randn(ring.ring_k.shape, device=dev, generator=g) / 2).bfloat16())
        ring.ring_v.copy_((torch.randn(ring.ring_v.shape, device=dev, generator=g) / 2).half())
        xs = torch.randn(512, HIDDEN, device=dev, generator=g).bfloat16()
        cos = torch.ones(1, 1, 64, device=dev); sin = torch.zeros(1, 1, 64, device=dev)
        for i in range(4):
            ops.decode_step(xs, w, cos, sin, ring.ring_k[0], ring.ring_v[0], 250 + i)
    torch.cuda.synchronize()
    assert ops.read_status(ops.default_status(dev)) == 0
    print(f"profile case {which}: done")


def run_extra_workload(args) -> None:
    """Secondary benchmark configurations, one JSON line each (single GPU; not the headline line):
    longclip = config 4 (16 clips x 2500 frames, banded attention alone, rotated BF16 q,k / FP16 v resident);
    stream   = config 5 (4096 streams x 500 one-frame steps x 8 layers from an empty 250-slot ring)."""
    import fast_mimi_b200 as fm
    from fast_mimi_b200 import ops
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    stream = torch.cuda.current_stream()
    g = torch.Generator(device=dev).manual_seed(0)
    if args.workload == "stack":
        run_stack(args, dev, peaks, stream, g)
        return
    if args.workload == "streamlayer":
        # config 5's step through WHOLE transformer layers (LayerNorms, projections, ring decode, MLP; all on this
        # library's kernels): 4096 streams x 8 layers, one new frame per stream, full 250-slot rings
        S, L = 4096, 8
        layers = [fm.MimiTransformerLayerB200(layer_idx=l).to(dev) for l in range(L)]
        ring = fm.MimiKVRing(L, S, WINDOW, device=dev)
        ring.ring_k.copy_((torch.randn(ring.ring_k.shape[1:], device=dev, generator=g) / 2).bfloat16().expand_as(ring.ring_k))
        ring.ring_v.copy_((torch.randn(ring.ring_v.shape[1:], device=dev, generator=g) / 2).half().expand_as(ring.ring_v))
        ring._cumulative_lengths = [WINDOW] * L
        x = torch.randn(S, 1, HIDDEN, device=dev, generator=g)

        def one_step(pos):
            cs = fm.rope_tables(torch.tensor([[pos]], device=dev))
            h = x
            with torch.no_grad():
                for layer in layers:
                    h, _ = layer(h, None, ring, cs, False)
            return h

        n_warm = max(args.warmup, 3)
        for i in range(n_warm):
            one_step(WINDOW + i)
        torch.cuda.synchronize()
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
        steps = min(args.steps, 50)
        a.record(stream)
        for i in range(steps):
            one_step(WINDOW + n_warm + i)
        b.record(stream)
        torch.cuda.synchronize()
        fm.check_status()
        ms = a.elapsed_time(b) / steps
        ring_bytes = S * L * (2 * WINDOW * 512 * 2)
        print(json.dumps({"metric": "transformer-layer frames/s (streaming)", "value": S * L / (ms / 1e3), "unit": "frames/s",
                          "n_gpus": 1, "steps": steps, "ms_per_step": ms, "dtype": "fp16 operands, bf16 / fp16 ring, fp32 residual stream",
                          "data": "synthetic",
                          "config": {"workload": "streaming decode through whole transformer layers (benchmark config 5's step)",
                                     "streams": S, "layers": L, "ring_slots": WINDOW},
                          "ring_gbs": ring_bytes / (ms / 1e3) / 1e9, "frac_hbm_ring_only": ring_bytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"]}))
        return
    if args.workload == "rvq":
        # the quantiser that follows the encoder transformer: config 3's batch after the stride-2 downsample,
        # 512 clips x 125 frames = 64 000 vectors of 256 dimensions, 8 codebooks of 2048 entries
        rows, layers = CLIPS * FRAMES // 2, 8
        books = ops.RVQCodebooks(torch.randn(layers, 2048, 256, device=dev, generator=g)
                                 * (0.6 ** torch.arange(layers, device=dev, dtype=torch.float32))[:, None, None])
        # embeddings [rows, 512] -> the quantiser's 1 x 1 input projection (512 -> 256, split-precision tensor-core
        # product) -> eight layers of search; the projection is inside the timed region
        emb = torch.randn(rows, HIDDEN, device=dev, generator=g) * 1.5
        proj = ops.split_half((torch.randn(256, HIDDEN, device=dev, generator=g) / HIDDEN ** 0.5).contiguous())
        x = ops.linear_split(emb, proj)
        for _ in range(max(args.warmup, 3)):
            codes, cand = ops.rvq_encode(ops.linear_split(emb, proj), books, return_candidates=True)
        torch.cuda.synchronize()
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True); c = torch.cuda.Event(enable_timing=True)
        ms_proj = 0.0
        a.record(stream)
        for _ in range(args.steps):
            ops.rvq_encode(ops.linear_split(emb, proj), books)
        b.record(stream)
        for _ in range(args.steps):
            ops.linear_split(emb, proj)
        c.record(stream)
        torch.cuda.synchronize()
        ops.check_status(dev)
        ms = a.elapsed_time(b) / args.steps
        ms_proj = b.elapsed_time(c) / args.steps
        flop = rows * layers * 2 * 2048 * 256
        nbytes = rows * layers * (2 * 32 * 16 + 256 * (2 + 4 + 4 + 2))      # candidate records written + read, residual in both types
        print(json.dumps({"metric": "quantised vectors/s", "value": rows / (ms / 1e3), "unit": "vectors/s", "n_gpus": 1,
                          "steps": args.steps, "ms_per_step": ms, "dtype": "fp16 pre-selection, fp32 decision", "data": "synthetic",
                          "config": {"workload": "residual vector quantisation encode, 8 codebooks x 2048 x 256",
                                     "vectors": rows, "layers": layers},
                          "tensor_tflops": flop / (ms / 1e3) / 1e12, "gbs": nbytes / (ms / 1e3) / 1e9,
                          "frac_hbm": nbytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"],
                          "input_projection_ms": ms_proj, "scores_in_memory": False,
                          "exact_evaluations_per_vector_layer": float(cand.float().mean())}))
        return
    if args.workload == "longclip":
        B, T = 16, 2500
        sets = []
        for _ in range(3):      # three input sets in rotation: 492 MB, so no set survives in the 126 MB L2
            q = (torch.randn(B, T, 512, device=dev, generator=g) / 8).bfloat16()
            k = (torch.randn(B, T, 512, device=dev, generator=g) / 8).bfloat16()
            v = (torch.randn(B, T, 512, device=dev, generator=g) / 8).half()
            sets.append((q, k, v))
        out = torch.empty_like(sets[0][2])
        for i in range(max(args.warmup, 3)):
            ops.band_attention_prefill(*sets[i % 3], window=WINDOW, out=out)
        torch.cuda.synchronize()
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for i in range(args.steps):
            ops.band_attention_prefill(*sets[i % 3], window=WINDOW, out=out)
        b.record(stream)
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        flop = B * 2048 * pairs(T)
        nbytes = 4 * B * T * 512 * 2
        gbs = nbytes / (ms / 1e3) / 1e9
        print(json.dumps({"metric": "attention frames/s", "value": B * T / (ms / 1e3), "unit": "frames/s", "n_gpus": 1,
                          "steps": args.steps, "ms_per_step": ms, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": "long-clip banded attention (benchmark config 4), one layer call",
                                     "clips": B, "frames": T, "window": WINDOW,
                                     "l2": "three input sets in rotation (492 MB)"},
                          "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                       "frac": gbs / peaks["hbm_gbs"], "kernel": "band_attn_long_kernel",
                                       "tensor_tflops": flop / (ms / 1e3) / 1e12}}))
        return
    # stream: the whole of config 5
    S, L, STEPS = 4096, 8, 500
    ring = fm.MimiKVRing(L, S, WINDOW, device=dev)
    ws = [(torch.randn(1536, HIDDEN, device=dev, generator=g) * 0.02).bfloat16() for _ in range(L)]
    xs = [torch.randn(S, HIDDEN, device=dev, generator=g).bfloat16() for _ in range(4)]
    pos = torch.arange(STEPS, device=dev, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2, device=dev, dtype=torch.int64).float() / 64))
    emb = torch.cat((torch.outer(pos, inv),) * 2, -1)
    cos, sin = emb.cos().contiguous(), emb.sin().contiguous()
    qws = torch.empty_like(xs[0]); out = torch.empty(S, HIDDEN, device=dev, dtype=torch.float32)
    status = ops.new_status(dev)

    plans = [[ops.DecodePlan(xs[j], ws[l], ring.ring_k[l], ring.ring_v[l], q_workspace=qws, out=out, status=status)
              for j in range(4)] for l in range(L)]
    cos3, sin3 = cos.view(STEPS, 1, 1, 64), sin.view(STEPS, 1, 1, 64)

    PARITY_STEPS, PARITY_LAYERS, PARITY_STREAMS = (0, 249, 250, 499), (0, L - 1), 32

    def run_all(capture=None):
        for t in range(STEPS):
            c, s_ = cos3[t], sin3[t]
            for l in range(L):
                plans[l][(t + l) & 3].step(t, c, s_)
                if capture is not None and t in PARITY_STEPS and l in PARITY_LAYERS:
                    capture[(t, l)] = out[:PARITY_STREAMS].clone()

    run_all()                      # warm-up pass (the ring is simply overwritten by the timed pass)
    torch.cuda.synchronize()
    a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
    a.record(stream)
    run_all()
    b.record(stream)
    torch.cuda.synchronize()
    ops.check_status(status=status)
    ms = a.elapsed_time(b)
    # Parity of this workload's own steps (an untimed third pass captures them): the first streams at the first
    # step, the last step of the fill, the first wrapped step and the last step, first and last layer, against the
    # CPU oracle driven through the same 500 steps with the reference's concatenate-and-crop cache.
    parity = None
    if not args.no_cpu:
        from oracle import mimi_attention_oracle as O
        got: dict = {}
        run_all(got)
        torch.cuda.synchronize()
        eye = torch.eye(HIDDEN)
        worst = 0.0
        for l in PARITY_LAYERS:
            wq, wk, wv = ws[l].float().cpu().chunk(3, 0)
            cache = O.KVCacheOracle()
            xs_cpu = [x_[:PARITY_STREAMS].float().cpu() for x_ in xs]
            for t in range(STEPS):
                want = O.attention_forward(xs_cpu[(t + l) & 3][:, None], wq, wk, wv, eye, cache=cache)
                if t in PARITY_STEPS:
                    worst = max(worst, O.rel_l2(got[(t, l)].cpu(), want.view(PARITY_STREAMS, HIDDEN)))
        parity = {"rel_l2_max": worst, "streams": PARITY_STREAMS, "steps": list(PARITY_STEPS), "layers": list(PARITY_LAYERS),
                  "tolerance": 2e-3, "ok": worst <= 2e-3}
    rows = sum(min(t + 1, WINDOW) for t in range(STEPS))
    nbytes = S * L * (rows * 2 * 512 * 2 + STEPS * (2048 + 1024 + 2048)) + STEPS * L * 1536 * 512 * 2
    gbs = nbytes / (ms / 1e3) / 1e9
    print(json.dumps({"metric": "attention frames/s", "value": S * STEPS * L / (ms / 1e3), "unit": "frames/s", "n_gpus": 1,
                      "steps": STEPS, "ms_total": ms, "ms_per_step": ms / STEPS, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "streaming decode (benchmark config 5), 500 steps from an empty ring",
                                 "streams": S, "layers": L, "ring_slots": WINDOW, "ring_gb": ring.bytes() / 1e9},
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                   "frac": gbs / peaks["hbm_gbs"], "kernel": "qkv_rope_gemm_kernel + ring_decode_attn_kernel",
                                   "algorithmic_bytes": nbytes}, "parity": parity}))


def run_stack(args, dev, peaks, stream, g) -> None:
    """Whole transformer layers (LayerNorm, projection + RoPE + banded attention in one kernel, o_proj, LayerNorm,
    MLP; six launches per layer, as MimiTransformerLayerB200 issues them) over config 3's batch: 512 clips x 250 frames x 16 layers, FP32 residual stream,
    FP16 tensor-core operands.  One JSON line with per-kernel CUDA-event times and rooflines."""
    from fast_mimi_b200 import ops
    rows = CLIPS * FRAMES
    x0 = torch.randn(CLIPS, FRAMES, HIDDEN, device=dev, generator=g)
    mk = lambda *shape, std: (torch.randn(*shape, device=dev, generator=g) * std).half()
    layers = [{"qkv": mk(1536, HIDDEN, std=0.04), "o": mk(HIDDEN, HIDDEN, std=0.04), "fc1": mk(2048, HIDDEN, std=0.04),
               "fc2": mk(HIDDEN, 2048, std=0.02), "ln1w": torch.ones(HIDDEN, device=dev), "ln1b": torch.zeros(HIDDEN, device=dev),
               "ln2w": torch.ones(HIDDEN, device=dev), "ln2b": torch.zeros(HIDDEN, device=dev),
               "s1": torch.full((HIDDEN,), 0.01, device=dev), "s2": torch.full((HIDDEN,), 0.01, device=dev)}
              for _ in range(LAYERS)]
    pos = torch.arange(FRAMES, device=dev, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2, device=dev, dtype=torch.int64).float() / 64))
    emb = torch.cat((torch.outer(pos, inv),) * 2, -1)
    cos, sin = emb.cos()[None].contiguous(), emb.sin()[None].contiguous()
    xa, xb = x0.clone(), torch.empty_like(x0)
    h = torch.empty(x0.shape, dtype=torch.float16, device=dev)
    core = torch.empty_like(h)
    gbuf = torch.empty(CLIPS, FRAMES, 2048, dtype=torch.float16, device=dev)
    status = ops.new_status(dev)
    names = ["layernorm512 (1)", "attn_fused_clip (projection + RoPE + attention)", "linear_gemm o_proj", "layernorm512 (2)",
             "linear_gemm fc1+gelu", "linear_gemm fc2"]

    def layer(p, x_in, x_mid, x_out, ev=None):
        def mark():
            if ev is not None:
                e = torch.cuda.Event(enable_timing=True); e.record(stream); ev.append(e)
        mark(); ops.layer_norm(x_in, p["ln1w"], p["ln1b"], out=h)
        mark(); ops.attention_prefill(h, p["qkv"], cos, sin, window=WINDOW, scale=0.125, out=core, status=status)
        mark(); ops.linear(core, p["o"], scale=p["s1"], residual=x_in, out=x_mid, status=status)
        mark(); ops.layer_norm(x_mid, p["ln2w"], p["ln2b"], out=h)
        mark(); ops.linear(h, p["fc1"], activation="gelu", out=gbuf, status=status)
        mark(); ops.linear(gbuf, p["fc2"], scale=p["s2"], residual=x_mid, out=x_out, status=status)
        mark()

    def step(evs=None):
        a, b = xa, xb
        for p in layers:
            ev = [] if evs is not None else None
            layer(p, a, b, a, ev)      # x_mid in b, result back in a
            if evs is not None:
                evs.append(ev)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    evs: list = []
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index or 0) as clocks:
        e0.record(stream)
        for _ in range(args.steps):
            step(evs)
        e1.record(stream)
        torch.cuda.synchronize()
    if ops.read_status(status) != 0:
        raise SystemExit("stack: a bounded device wait timed out")
    ms = e0.elapsed_time(e1) / args.steps
    per = [statistics.mean(ev[i].elapsed_time(ev[i + 1]) for ev in evs) for i in range(6)]
    flops = [0, 2 * 512 * 1536 + 2048 * pairs(FRAMES) / FRAMES, 2 * 512 * 512, 0, 2 * 512 * 2048, 2 * 512 * 2048]
    nbytes = [2048 + 1024, 1024 + 1024, 1024 + 2048 + 2048, 2048 + 1024, 1024 + 4096, 4096 + 2048 + 2048]
    kernels = []
    for n, t, f, b in zip(names, per, flops, nbytes):
        kernels.append({"kernel": n, "ms": t, "share": t / sum(per), "tflops": rows * f / (t / 1e3) / 1e12,
                        "gbs": rows * b / (t / 1e3) / 1e9, "frac_hbm": rows * b / (t / 1e3) / 1e9 / peaks["hbm_gbs"],
                        "frac_tensor": rows * f / (t / 1e3) / 1e12 / peaks["bf16_tflops"]})
    total_flop = rows * sum(flops) * LAYERS
    print(json.dumps({"metric": "transformer-layer frames/s", "value": rows * LAYERS / (ms / 1e3), "unit": "frames/s",
                      "n_gpus": 1, "steps": args.steps, "ms_per_step": ms, "dtype": "fp16 operands, fp32 accumulate and residual stream",
                      "data": "synthetic",
                      "config": {"workload": "whole transformer layers over benchmark config 3's batch", "clips": CLIPS,
                                 "frames": FRAMES, "layers": LAYERS, "launches_per_layer": 6,
                                 "l2": "per-layer tensors (0.26-0.52 GB each) exceed the 126 MB L2"},
                      "step_tflops": total_flop / (ms / 1e3) / 1e12, "frac_tensor": total_flop / (ms / 1e3) / 1e12 / peaks["bf16_tflops"],
                      "gpu_launches": args.steps * LAYERS * 6, "kernels": kernels, "clocks": clocks.summary()}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true", help="skip the streaming-decode measurement")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU oracle baseline")
    ap.add_argument("--profile-case", choices=["prefill", "fused", "chunk", "decode", "layer", "longclip", "rvq"],
                    help="run a small case for ncu and exit")
    ap.add_argument("--workload", default="prefill", choices=["prefill", "longclip", "stream", "streamlayer", "stack", "rvq"],
                    help="prefill = headline (config 3); longclip / stream = configs 4 / 5, stack = whole transformer layers, rvq = the quantiser after the encoder transformer; one extra JSON line each")
    args = ap.parse_args()
    if args.profile_case:
        profile_case(args.profile_case)
        return
    if args.workload != "prefill":
        run_extra_workload(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
