"""Benchmark of the NVFP4 MoE layer (router + routed experts + shared expert +
combine) through the library's C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1 (default): the decode-shaped layer microbenchmark — hidden 2048, 512
experts, top-10, intermediate 512, shared expert 512, T = 128 tokens per step,
uniform-random routing, NVFP4 weights ~ N(0, 0.02).  Each step runs one layer
forward; successive steps rotate over several independent layer weight sets
and inputs so that no step finds its weights in L2.  The line also carries the
sweep over T in {1, 8, 16, 32, 64}, the 16384-token Zipf-skewed prefill layer,
the MTP draft layer's BF16-expert MoE and the 48-layer decode stack
(x <- x + MoE(RMSNorm(x)), eager and as one CUDA graph, at T = 128 and at 1 and 8
tokens) under "also".  "e2e" is the same step fed from pinned host memory with
the result copied back, copies on their own streams.

N > 1 (launched by torchrun, one rank per GPU): the expert-parallel prefill
layer, T = 32768 tokens per step sharded by rank (strong scaling).  Default
exchange: kernels store into peer memory over NVLink (NCCL carries only the
expert ids and one barrier), the most used experts replicated on every GPU;
--exchange rows is the all-to-all of rows over NCCL with 512/N experts per GPU.

--impl reference times the reference's CPU formulation of the layer (the CPU
oracle's restatement of the reference's host-side MoE) on the host cores.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HS, E, K_TOP, MOE_IS, SHARED_IS = 2048, 512, 10, 512, 512
EXPERT_BYTES = 1_048_576 + 131_072 + 524_288 + 65_536 + 16      # codes + scales + 4 scalars
LAYER_FIXED_BYTES = 2_097_152 + 6_295_552                         # router + bf16 shared expert
GU_EXPERT_BYTES = 1_048_576 + 131_072                             # gate/up codes + scales
# 2*128*256*64 flops per 129 clocks per SM (measured), 148 SMs, 1965 MHz
NVFP4_MMA_ISSUE_PEAK_TFLOPS = 2 * 128 * 256 * 64 / 129 * 148 * 1.965e9 / 1e12


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons while a timed region runs: through NVML from
    a thread (every few milliseconds, so that even a short region is covered), or, without
    the NVML module, through an `nvidia-smi -lms` child.  Read-only queries."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index=0, period_s=0.004):
        self.index, self.rows, self.proc, self.period = index, [], None, period_s
        self.stop = threading.Event()
        self.thread = None
        self.nvml = None

    def _nvml_sample(self):
        nv, h = self.nvml
        bits = (nv.nvmlClocksThrottleReasonHwSlowdown, nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                nv.nvmlClocksThrottleReasonSwThermalSlowdown, nv.nvmlClocksThrottleReasonSwPowerCap)
        try:
            sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
            mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
            self.rows.append([str(sm), str(self.max_mhz)] + ["Active" if mask & b else "Not Active" for b in bits])
        except Exception:   # a failed query is a missing sample, nothing more
            pass

    def _nvml_loop(self):
        while not self.stop.is_set():
            self._nvml_sample()
            self.stop.wait(self.period)

    def __enter__(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.nvml = (nv, h)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.nvml is not None:
            self._nvml_sample()   # the region has just ended: the GPU is still at its load clocks
        self.stop.set()
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        elif self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for r in list(self.rows):
            try:
                sm.append(int(float(r[0])))
                mx = max(mx, int(float(r[1])))
            except (ValueError, IndexError):
                continue
            for name, v in zip(self.NAMES, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=mx or None, reasons=sorted(reasons),
                    samples=len(sm))


def time_steps(torch, fn, steps, warmup, barrier=None, finish=None, repeats=1):
    """W untimed steps, then exactly K timed steps between CUDA events on the
    current stream, with a synchronise (and barrier) on both sides.  With repeats > 1 the
    K-step region is timed that many times back to back and the list of per-step times (ms)
    is returned instead of one number."""
    for i in range(warmup):
        fn(i)
    out = []
    n = warmup
    for _ in range(max(1, repeats)):
        torch.cuda.synchronize()
        if barrier:
            barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(steps):
            fn(n + i)
        n += steps
        if finish:      # e.g. make the timing stream wait for copies still running on other streams
            finish()
        t1.record()
        torch.cuda.synchronize()
        if barrier:
            barrier()
        out.append(t0.elapsed_time(t1) / steps)
    return out if repeats > 1 else out[0]


def spread(ms_list):
    """min / median / p95 of repeated timings of the same K-step region (ms per step)."""
    v = sorted(ms_list)
    n = len(v)
    return dict(repeats=n, min=v[0], median=v[n // 2] if n % 2 else 0.5 * (v[n // 2 - 1] + v[n // 2]),
                p95=v[min(n - 1, int(round(0.95 * (n - 1))))], max=v[-1])


def unique_experts(torch, fwd, T):
    ids = fwd.region("expert_ids", torch.int32, T * K_TOP)
    return int(torch.unique(ids).numel())


def layer_bytes(U, T):
    return U * EXPERT_BYTES + LAYER_FIXED_BYTES + 2 * T * HS * 2


def run_decode_point(torch, q4t, layers, T, steps, warmup, n_inputs=8, with_e2e=False, with_stages=False, repeats=1):
    syn = importlib.import_module("qwen4-thor_b200.synthetic")
    xs = [syn.make_x(T, HS, seed=100 + i) for i in range(n_inputs)]
    fwds = [q4t.MoEForward(l, T, K_TOP) for l in layers]
    y = torch.empty((T, HS), dtype=torch.bfloat16, device="cuda")
    counter = {"launches": 0}

    def step(i):
        fwds[i % len(fwds)](xs[i % n_inputs], y)

    timing = None
    if repeats > 1:     # the K-step region repeated: the median is the reported time
        timing = spread(time_steps(torch, step, steps, warmup, repeats=repeats))
        ms = timing["median"]
    else:
        ms = time_steps(torch, step, steps, warmup)
    fwds[0].status()
    # distinct experts per step (algorithmic bytes), averaged over the rotation
    us = []
    for i in range(min(len(fwds) * 2, 8)):
        step(i)
        torch.cuda.synchronize()
        us.append(unique_experts(torch, fwds[i % len(fwds)], T))
    U = sum(us) / len(us)
    out = dict(T=T, ms_per_step=ms, tokens_per_s=T / (ms * 1e-3), unique_experts=U,
               layer_bytes=layer_bytes(U, T), layer_gbs=layer_bytes(U, T) / (ms * 1e-3) / 1e9)
    if timing:
        out["ms_per_step_spread"] = timing
    if with_stages:
        q4t.stage_timing(True)
        acc = {}
        n = max(steps, 8)
        for i in range(n):
            step(i)
            for kname, v in q4t.stage_timing_read().items():
                acc[kname] = acc.get(kname, 0.0) + v
        q4t.stage_timing(False)
        out["stage_ms"] = {kname: v / n for kname, v in acc.items()}
    if with_e2e:
        # Every step copies its input from pinned host memory and its result back.  The copies
        # run on their own streams with two buffers each way, so the input of step i+1 and the
        # result of step i-1 move while step i computes; the timed region ends only when the
        # last result has reached the host.
        hx = [x.cpu().pin_memory() for x in xs]
        hy = [torch.empty((T, HS), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        dx = [torch.empty((T, HS), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        dy = [torch.empty((T, HS), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        main, s_in, s_out = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        for e in ev_done + ev_out:
            e.record(main)

        def step_e2e(i):
            b = i & 1
            s_in.wait_event(ev_done[b])            # the forward that last read dx[b] is over
            with torch.cuda.stream(s_in):
                dx[b].copy_(hx[i % n_inputs], non_blocking=True)
                ev_in[b].record(s_in)
            main.wait_event(ev_in[b])
            main.wait_event(ev_out[b])             # dy[b] has been copied out
            fwds[i % len(fwds)](dx[b], dy[b])
            ev_done[b].record(main)
            s_out.wait_event(ev_done[b])
            with torch.cuda.stream(s_out):
                hy[b].copy_(dy[b], non_blocking=True)
                ev_out[b].record(s_out)

        def drain():
            main.wait_event(ev_out[0])
            main.wait_event(ev_out[1])

        if repeats > 1:
            sp = spread(time_steps(torch, step_e2e, steps, warmup, finish=drain, repeats=repeats))
            ms_e = sp["median"]
        else:
            sp, ms_e = None, time_steps(torch, step_e2e, steps, warmup, finish=drain)
        out["e2e"] = dict(value=T / (ms_e * 1e-3), unit="tokens/s", ms_per_step=ms_e,
                          h2d_bytes_per_step=T * HS * 2, d2h_bytes_per_step=T * HS * 2)
        if sp:
            out["e2e"]["ms_per_step_spread"] = sp
    del fwds
    return out


def run_prefill_point(torch, q4t, T, steps, warmup, seed=7, repeats=5):
    syn = importlib.import_module("qwen4-thor_b200.synthetic")
    layer = syn.device_layer(q4t, E, HS, MOE_IS, SHARED_IS, seed=seed, zipf_s=1.1)
    xs = [syn.make_x(T, HS, seed=200 + i, bias_column=True) for i in range(2)]
    fwd = q4t.MoEForward(layer, T, K_TOP)
    y = torch.empty((T, HS), dtype=torch.bfloat16, device="cuda")
    sp = spread(time_steps(torch, lambda i: fwd(xs[i % 2], y), steps, warmup, repeats=max(1, repeats)))
    ms = sp["median"]
    fwd.status()
    counts = fwd.routed_region("counts", torch.int32, E).float()
    q4t.stage_timing(True)
    acc = {}
    for i in range(3):
        fwd(xs[i % 2], y)
        for kname, v in q4t.stage_timing_read().items():
            acc[kname] = acc.get(kname, 0.0) + v / 3
    q4t.stage_timing(False)
    flops = 6.0 * T * K_TOP * HS * MOE_IS
    out = dict(T=T, ms_per_step=ms, ms_per_step_spread=sp, tokens_per_s=T / (ms * 1e-3),
               routed_tflops=flops / (ms * 1e-3) / 1e12,
               rows_per_expert_max=float(counts.max()), rows_per_expert_mean=float(counts.mean()),
               stage_ms=acc, routing="zipf(s=1.1) bias on router column 0")
    del fwd, layer
    return out


def run_mtp_bf16_point(torch, q4t, Ts=(1, 4, 8), steps=20, warmup=3):
    """The MTP draft layer's MoE (BF16 routed experts, src/mtp/moe_bf16.cu of the reference) at the
    reference's shapes: hidden 2560, 512 experts of intermediate 640, top-10.  A decode-sized step
    streams the selected experts' BF16 weights once, so the bound is HBM."""
    syn = importlib.import_module("qwen4-thor_b200.synthetic")
    E_, hs, is_, sis = 512, 2560, 640, 640
    g = torch.Generator(device="cuda").manual_seed(20260921 + 77)
    gu = torch.empty((E_, 2 * is_, hs), dtype=torch.bfloat16, device="cuda")
    down = torch.empty((E_, hs, is_), dtype=torch.bfloat16, device="cuda")
    for e0 in range(0, E_, 64):     # in slices: the fp32 staging of all 512 experts would take 10 GB
        gu[e0:e0 + 64] = (torch.randn((64, 2 * is_, hs), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
        down[e0:e0 + 64] = (torch.randn((64, hs, is_), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    extra = syn.device_layer(q4t, E_, hs, 128, sis, seed=20260921 + 78)   # router and shared expert of the layer
    peaks = load_peaks()
    out = []
    for T in Ts:
        moe = q4t.Bf16MoE(gu, down, extra, T, K_TOP)
        xs = [syn.make_x(T, hs, seed=300 + i) for i in range(8)]
        y = torch.empty((T, hs), dtype=torch.bfloat16, device="cuda")
        ms = time_steps(torch, lambda i: moe.forward(xs[i % 8], y), steps, warmup)
        ws = moe.ws
        fl = q4t.forward_ws_layout(T, K_TOP, hs, is_, sis, E_)
        ids = ws[fl.expert_ids:fl.expert_ids + T * K_TOP * 4].view(torch.int32)
        U = int(torch.unique(ids).numel())
        nbytes = U * 3 * is_ * hs * 2 + (E_ + 3 * sis + 1) * hs * 2
        out.append(dict(T=T, ms_per_step=ms, tokens_per_s=T / (ms * 1e-3), unique_experts=U, bytes=nbytes,
                        gbs=nbytes / (ms * 1e-3) / 1e9, hbm_frac_of_measured=nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]))
    del gu, down
    torch.cuda.empty_cache()
    return dict(workload="MTP draft layer MoE, BF16 routed experts, hidden 2560, 512 experts x intermediate 640, top-10",
                l2="each step selects its own experts; 7 to 300 MB of weights per step, inputs rotated", points=out)


def run_dense_fp4_point(torch, q4t, M, N, Kd, secs=0.3):
    """A dense NVFP4 GEMM of M x N x K through q4t_fp4_gemm (bf16 output, random codes): what the
    block-scaled tensor-core mainloop of this library sustains when every row tile is full."""
    import ctypes as C
    L = q4t.load()
    w = torch.randint(0, 256, (N, Kd // 2), dtype=torch.uint8, device="cuda")
    a = torch.randint(0, 256, (M, Kd // 2), dtype=torch.uint8, device="cuda")
    wsf = torch.full((L.q4t_sf_buffer_size(N, Kd),), 0x38, dtype=torch.uint8, device="cuda")
    asf = torch.full((L.q4t_sf_buffer_size(M, Kd),), 0x38, dtype=torch.uint8, device="cuda")
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def f(_i=0):
        q4t.check(L.q4t_fp4_gemm(w.data_ptr(), wsf.data_ptr(), a.data_ptr(), asf.data_ptr(), out.data_ptr(), 1, M, N, Kd,
                                 C.c_float(1.0), C.c_float(1.0), st))

    ms1 = time_steps(torch, f, 3, 3)
    iters = max(5, int(secs * 1e3 / max(ms1, 1e-3)))
    ms = time_steps(torch, f, iters, 0)
    return dict(M=M, N=N, K=Kd, ms=ms, tflops=2.0 * M * N * Kd / (ms * 1e-3) / 1e12, iters=iters)


def cpu_reference_run(q4t_layer_host, T, steps, warmup, bias_column=False, threads=None):
    """Times the CPU formulation (oracle 'test twin' mode: dequantise, fp32
    sequential dots, expf) on `threads` host threads (default: all); returns
    (tokens/s, ms, threads)."""
    from oracle import oracle as O
    import numpy as np
    if threads is not None:
        O.set_num_threads(threads)
    rng = np.random.default_rng(5)
    xf = rng.standard_normal((T, HS), dtype=np.float32)
    if bias_column:      # the column that carries the router's popularity bias
        xf[:, 0] = 1.0
    x = O.f32_to_bf16(xf)
    for _ in range(warmup):
        O.moe_forward(x, q4t_layer_host, K_TOP, 0, 0, 0)
    t0 = time.perf_counter()
    for _ in range(steps):
        O.moe_forward(x, q4t_layer_host, K_TOP, 0, 0, 0)
    dt = (time.perf_counter() - t0) / steps
    return T / dt, dt * 1e3, O.num_threads()


def host_layer_from_device(torch, dl):
    from oracle import oracle as O
    import numpy as np
    arrs = {}
    for n, t in dl.t.items():
        a = t.view(torch.int16).cpu().numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.cpu().numpy()
        arrs[n] = a
    return O.Layer(dl.E, dl.hs, dl.moe_is, dl.shared_is, **arrs)


def pick_cpu_tokens(layer_host, budget_s=4.0):
    """Largest T <= 128 whose CPU step is expected to stay near budget_s."""
    _, ms8, _ = cpu_reference_run(layer_host, 8, 1, 0)
    per_tok = ms8 / 8.0 / 1e3
    T = int(max(1, min(128, budget_s / max(per_tok, 1e-6))))
    return T


# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up GEMM launch at T = 128 divided by
# the experts that launch touched (ncu --set full capture, summarised under profiles/)
GU_DRAM_BYTES_PER_EXPERT = 567.25e6 / 467.5


def run_stack_point(torch, q4t, syn, layers, n_layers, T, passes, layer_bytes):
    """Config 3: n_layers layers with independent weights, x <- bf16(x + MoE(RMSNorm(x))), T tokens.
    One pass = the whole stack; timed eagerly and, when capture works, as one CUDA graph."""
    t_build = time.time()
    while len(layers) < n_layers:
        layers.append(syn.device_layer(q4t, E, HS, MOE_IS, SHARED_IS, seed=20260921 + 1000 + len(layers)))
    build_s = time.time() - t_build
    stack = q4t.DecodeStack(layers[:n_layers], T, K_TOP)
    x0 = syn.make_x(T, HS, seed=4242)
    x = x0.clone()

    def one_pass(_i=0):
        x.copy_(x0)
        stack(x)

    ms = time_steps(torch, one_pass, passes, 2)
    out = dict(layers=n_layers, tokens=T, build_s=build_s, ms_per_pass=ms, us_per_layer=ms * 1e3 / n_layers,
               layer_tokens_per_s=T * n_layers / (ms * 1e-3),
               hbm_frac_of_measured=layer_bytes * n_layers / (ms * 1e-3) / 1e9 / load_peaks()["hbm_gbs"],
               weights_gb=n_layers * 0.906, graph=None)
    try:   # the same pass as one CUDA graph (side-stream fork/join and chained launches are captured with it)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            one_pass()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                one_pass()
        torch.cuda.current_stream().wait_stream(side)
        x_ref = x.clone()
        ms_g = time_steps(torch, lambda i: graph.replay(), passes, 2)
        same = bool(torch.equal(x.view(torch.int16), x_ref.view(torch.int16)))
        out["graph"] = dict(ms_per_pass=ms_g, us_per_layer=ms_g * 1e3 / n_layers, replay_equals_eager=same,
                            hbm_frac_of_measured=layer_bytes * n_layers / (ms_g * 1e-3) / 1e9 / load_peaks()["hbm_gbs"])
    except Exception as exc:   # capture is optional: report why it was not measured
        out["graph"] = dict(error=str(exc).splitlines()[0][:200])
    return out


def main_single(args):
    import torch
    q4t = importlib.import_module("qwen4-thor_b200")
    syn = importlib.import_module("qwen4-thor_b200.synthetic")
    q4t.load()
    torch.cuda.set_device(0)
    peaks = load_peaks()
    if args.prefill_tokens > 0:
        print(json.dumps(dict(prefill=run_prefill_point(torch, q4t, args.prefill_tokens, args.steps, args.warmup))))
        return
    n_layers = 1 if args.impl == "reference" else args.layers
    multi_ref = args.impl == "reference" and args.gpus > 1   # the CPU arm of the expert-parallel workload
    layers = [syn.device_layer(q4t, E, HS, MOE_IS, SHARED_IS, seed=20260921 + (4000 if multi_ref else 1000 + i),
                               zipf_s=1.1 if multi_ref else None) for i in range(n_layers)]

    if args.impl == "reference":
        if multi_ref:   # the launcher pins every rank to one OpenMP thread; this arm is alone on the host
            from oracle import oracle as O
            O.set_num_threads(os.cpu_count() or 1)
        host_layer = host_layer_from_device(torch, layers[0])
        T = pick_cpu_tokens(host_layer)
        tps, ms, threads = cpu_reference_run(host_layer, T, args.steps, min(args.warmup, 1), bias_column=multi_ref)
        line = dict(impl="reference", metric="moe_layer_tokens_per_s", value=tps, unit="tokens/s", n_gpus=args.gpus,
                    steps=args.steps, warmup=min(args.warmup, 1), ms_per_step=ms, higher_is_better=True,
                    scaling="strong" if multi_ref else "weak", vs_baseline=None,
                    dtype="nvfp4 (e2m1 x ue4m3) weights and activations, fp32 accumulate",
                    data="synthetic",
                    config=dict(workload=("prefill MoE layer with the Zipf(1.1) router of the expert-parallel workload, "
                                          "hs=2048 E=512 top-10 is=512 shared=512, one host" if multi_ref else
                                          "decode-shaped MoE layer, hs=2048 E=512 top-10 is=512 shared=512"), tokens=T),
                    cpu_baseline=dict(value=tps, unit="tokens/s", cores=threads, kind="port",
                                      sample=f"one layer forward of {T} tokens per step"),
                    e2e=dict(value=tps, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
        print(json.dumps(line))
        return

    T = args.tokens
    if args.profile_range:   # for `ncu --profile-from-start off`: only the steps of the headline point are seen
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
    with ClockSampler(0) as clocks:
        main = run_decode_point(torch, q4t, layers, T, args.steps, args.warmup, with_e2e=not args.profile_range,
                                with_stages=not args.profile_range, repeats=args.repeats)
    if args.profile_range:
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps(dict(profile_range=True, tokens=T, ms_per_step=main["ms_per_step"])))
        return
    clk = clocks.summary()
    also = {}
    if not args.quick:
        sweep = []
        for t in (1, 8, 16, 32, 64):
            # these steps are 35-150 us long: a timed region of 50 is over in a few milliseconds, so it is
            # repeated (median reported) after a longer warm-up than the headline point needs
            r = run_decode_point(torch, q4t, layers, t, max(args.steps, 20), max(args.warmup, 20), with_stages=True,
                                 repeats=5)
            r["hbm_frac_of_measured"] = r["layer_gbs"] / peaks["hbm_gbs"]
            sweep.append(r)
        also["decode_sweep"] = sweep
        also["prefill_T16384"] = run_prefill_point(torch, q4t, 16384, max(3, min(args.steps, 10)), 3)
        pf = also["prefill_T16384"]
        pf["frac_of_4x_measured_bf16"] = pf["routed_tflops"] / (4 * peaks["bf16_tflops"])
        pf["frac_of_9pf_nominal"] = pf["routed_tflops"] / 9000.0
        # what this library's own block-scaled mainloop reaches on a dense problem of the gate/up
        # shape with every row tile full (no routing, no epilogue arithmetic): the practical
        # ceiling of the expert GEMMs on this GPU, measured beside the layer
        also["nvfp4_dense_gemm"] = run_dense_fp4_point(torch, q4t, 16384 * K_TOP, 2 * MOE_IS, HS)
        # the same expert-parallel batch the multi-GPU runs shard, on this one GPU
        ep1 = run_prefill_point(torch, q4t, 32768, max(3, min(args.steps, 10)), 3, seed=20260921 + 4000, repeats=3)
        also["ep_prefill_T32768_single_gpu"] = dict(metric="moe_ep_prefill_tokens_per_s", value=ep1["tokens_per_s"],
                                                    ms_per_step=ep1["ms_per_step"],
                                                    note="the workload of the --gpus N > 1 runs on one GPU "
                                                         "(strong-scaling reference)")

    # roofline of the dominant kernel (gate/up GEMM with fused SwiGLU + requantise)
    st = main["stage_ms"]
    R = T * K_TOP
    gu_bytes = main["unique_experts"] * GU_EXPERT_BYTES + R * (HS // 2 + HS // 16) + R * (MOE_IS // 2 + MOE_IS // 16)
    gu_gbs = gu_bytes / (st["gate_up_gemm"] * 1e-3) / 1e9
    roofline = dict(bound="hbm", kernel="gate_up_gemm (tcgen05 NVFP4 grouped GEMM + SwiGLU + requantise)",
                    achieved=gu_gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gu_gbs / peaks["hbm_gbs"],
                    peak_source=peaks["source"], traffic=GU_DRAM_BYTES_PER_EXPERT * main["unique_experts"],
                    traffic_source="ncu capture of one launch (567.25 MB at 467.5 experts), scaled by the experts touched",
                    algorithmic_bytes=gu_bytes,
                    kernel_ms=st["gate_up_gemm"],
                    layer=dict(achieved=main["layer_gbs"], frac=main["layer_gbs"] / peaks["hbm_gbs"],
                               frac_of_8tbs=main["layer_gbs"] / 8000.0, bytes=main["layer_bytes"]))

    cpu = None
    if not args.no_cpu:
        from oracle import oracle as O
        host_layer = host_layer_from_device(torch, layers[0])
        all_threads = O.num_threads()
        Tc = pick_cpu_tokens(host_layer)
        tps, ms_c, threads = cpu_reference_run(host_layer, Tc, 2, 1)
        # the reference's loop nest as written runs on one thread: timed on a smaller sample
        T1 = max(1, min(8, Tc // 8))
        tps1, ms_1, _ = cpu_reference_run(host_layer, T1, 1, 1, threads=1)
        O.set_num_threads(all_threads)
        cpu = dict(value=tps, unit="tokens/s", cores=threads, kind="port",
                   sample=f"2 layer forwards of {Tc} tokens (oracle restatement of the reference's host-side MoE)",
                   single_thread=dict(value=tps1, unit="tokens/s", cores=1,
                                      sample=f"1 layer forward of {T1} tokens, one thread"))

    if not args.quick:
        also["mtp_bf16_moe"] = run_mtp_bf16_point(torch, q4t)
    if not args.quick and args.stack_layers > 0:   # last: the graph capture attempt must not disturb the rest
        also["stack"] = run_stack_point(torch, q4t, syn, layers, args.stack_layers, T, 5, main["layer_bytes"])
        # the same stack at decode-sized batches: eagerly these steps are close to what the host can
        # launch (12 calls per layer), as one CUDA graph they show the device time per layer
        by_t = {r["T"]: r for r in also.get("decode_sweep", [])}
        also["stack_decode_sized"] = [run_stack_point(torch, q4t, syn, layers, args.stack_layers, t, 5,
                                                      by_t[t]["layer_bytes"]) for t in (1, 8) if t in by_t]

    prefill_roofline = None
    if "prefill_T16384" in also:
        pf = also["prefill_T16384"]
        dense = also.get("nvfp4_dense_gemm") or {}
        prefill_roofline = dict(bound="tensor", workload="prefill MoE layer, T=16384, Zipf(1.1) router",
                                flops=6.0 * 16384 * K_TOP * HS * MOE_IS, achieved=pf["routed_tflops"], unit="TFLOP/s",
                                peak=4 * peaks["bf16_tflops"], peak_source="4 x measured dense bf16 (no NVFP4 peak is measured by the driver)",
                                frac=pf["routed_tflops"] / (4 * peaks["bf16_tflops"]),
                                frac_of_9pf_nominal=pf["routed_tflops"] / 9000.0,
                                # issue rate of the instruction itself, from a microbenchmark on this pool's B200s:
                                # one tcgen05.mma kind::mxf4nvf4 128x256x64 per 129 clocks per SM
                                nvfp4_mma_issue_peak_tflops=NVFP4_MMA_ISSUE_PEAK_TFLOPS,
                                frac_of_mma_issue_peak=pf["routed_tflops"] / NVFP4_MMA_ISSUE_PEAK_TFLOPS,
                                own_dense_nvfp4_gemm_tflops=dense.get("tflops"),
                                frac_of_own_dense_nvfp4_gemm=(pf["routed_tflops"] / dense["tflops"]) if dense.get("tflops") else None,
                                ms_per_step=pf["ms_per_step"], stage_ms=pf["stage_ms"])
    # router logits, top-k + permutation (one cluster launch), gather-quantise, gate/up, down, combine;
    # shared expert: gate|up with SwiGLU, down
    launches_per_step = 1 + 1 + 1 + 1 + 1 + 1 + 2
    line = dict(metric="moe_layer_tokens_per_s", value=main["tokens_per_s"], unit="tokens/s", n_gpus=1,
                steps=args.steps, warmup=args.warmup, ms_per_step=main["ms_per_step"], higher_is_better=True,
                scaling="weak", vs_baseline=None,
                dtype="nvfp4 (e2m1 x ue4m3, fp32 accumulate); bf16 router and shared expert", data="synthetic",
                config=dict(workload=f"decode-shaped MoE layer microbench, T={T}", hidden=HS, experts=E, top_k=K_TOP,
                            moe_intermediate=MOE_IS, shared_intermediate=SHARED_IS,
                            l2=f"{args.layers} layer weight sets (0.9 GB each) and 8 inputs rotated per step; one step touches ~840 MB > L2",
                            unique_experts_per_step=main["unique_experts"]),
                clocks=clk, e2e={k: v for k, v in main["e2e"].items() if k != "ms_per_step"},
                gpu_launches=launches_per_step * args.steps, roofline=roofline, prefill=prefill_roofline,
                cpu_baseline=cpu, ms_per_step_spread=main.get("ms_per_step_spread"), stage_ms=st, also=also)
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--exchange", default="peer", choices=["peer", "rows"],
                    help="multi-GPU only: peer-memory pull/push (default) or NCCL all-to-all of rows")
    ap.add_argument("--hot-experts", type=int, default=32,
                    help="multi-GPU peer exchange: experts replicated on every GPU (0 = none, interleaved sharding)")
    ap.add_argument("--quick", action="store_true", help="headline point only (no sweep, no prefill)")
    ap.add_argument("--repeats", type=int, default=10,
                    help="how many times the K-step timed region of the headline point is repeated (median reported)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--layers", type=int, default=4, help="independent layer weight sets rotated per step")
    ap.add_argument("--stack-layers", type=int, default=48,
                    help="layers of the decode-stack point (x <- x + MoE(RMSNorm(x)), T=128); 0 skips it")
    ap.add_argument("--tokens", type=int, default=128,
                    help="tokens per step of the headline point (128 = the benchmark's configuration)")
    ap.add_argument("--profile-range", action="store_true",
                    help="bracket the headline point's steps with cudaProfilerStart/Stop and print only its time "
                         "(for launch lists and captures taken with ncu --profile-from-start off)")
    ap.add_argument("--prefill-tokens", type=int, default=0,
                    help="run only the Zipf-skewed prefill layer at this many tokens and print its result")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and "RANK" not in os.environ:
        # not under torchrun: start one rank per GPU ourselves
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.gpus),
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29577"),
               os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    if world > 1 or args.gpus > 1:
        from importlib import import_module
        ep = import_module("qwen4-thor_b200.ep_bench")
        ep.main_multi(args)
        return
    main_single(args)


if __name__ == "__main__":
    main()
