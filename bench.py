"""Benchmark of the compressed-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (N = 1): single-layer decode attention over a compressed cache at the
Llama-3.1-8B layer shape - 32 query heads, 8 KV heads, head_dim 128, batch 1, context 32768 =
128 fp16 sink + 32512 tokens packed at 4-bit keys / 2-bit values + 128 fp16 recent tokens.
One STEP is that attention for the 32 layers of the model, each layer with its own cache, so the
working set (0.9 GB) is far larger than L2.  Synthetic seeded K/V/Q with the benchmark's
distributions stand in for model activations.

Printed JSON (one line): `value` = algorithmic HBM GB/s over all GPUs with everything resident in
HBM (CUDA-graph replay of the 32 launches, CUDA events); `e2e` = the same quantity through the
public cache API with host buffers (pinned host -> device copies of the new token's q/k/v and the
device -> host read of the result inside the timed region); `roofline` for the dominant kernel;
`cpu_baseline` = the reference's own per-step work (dense reassembly + float32 attention) restated on
the host cores; `secondary` = quantize+pack throughput in Mtokens/s.

`--impl reference` times that CPU restatement alone (no GPU work on its path).
With N > 1 (launched under torchrun) every rank owns an independent set of sequences: no data-path
collective, weak scaling, time = max over ranks.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# ---- workload constants (Llama-3.1-8B layer, 32K context, K4/V2) ----------------------------------------
LAYERS, HQ, HKV, D, CTX, SINK, RW = 32, 32, 8, 128, 32768, 128, 128
T_C = CTX - SINK - RW
# algorithmic bytes of one layer-step: packed codes + norms, fp16 sink/recent tokens, query in, result out
BYTES_PER_LAYER_STEP = HKV * T_C * (D * 4 // 8 + 4 + D * 2 // 8 + 4) + HKV * (SINK + RW) * 2 * D * 2 + HQ * D * 4
# the ncu summary of the decode kernel on this workload; its "DRAM traffic per launch" line feeds roofline.traffic
DECODE_PROFILE = "profiles/decode_direct_kernel_c1_k4v2_ctx32768.md"
WORKLOAD = "llama31_8b_layer_decode_attn_ctx32768_k4v2_sink128_rw128"
# quantize+pack: 4096-token chunks x 8 KV heads, K and V, fp16 in; bytes per (token, head): read 2*D*2, write codes + norms
QCHUNK = 4096


def ncu_traffic_bytes():
    """DRAM bytes (read + write) of one decode launch, as captured by ncu and written into the profile summary."""
    import re
    try:
        m = re.search(r"DRAM traffic per launch \(read \+ write\): ([0-9,]+) bytes", (ROOT / DECODE_PROFILE).read_text())
        return int(m.group(1).replace(",", "")) if m else None
    except OSError:
        return None


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU every 100 ms while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None
            return self
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self):
        nv = self._nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=1)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- the reference's per-step work, restated on the CPU ---------------------------------------------------
def cpu_reference_step_factory(layers: int, seed0: int = 1000):
    """Build `layers` reference-style caches on the host (oracle: quantize, dequantize -> dense middle) and
    return (step_fn, info).  step_fn() does, per layer, what the reference does per decode step: append the
    token, reassemble dense [sink | middle | recent] float32 K/V (cache.py:682-706) and run float32 GQA
    attention on it."""
    from mlx_turboquant_b200.codebook import get_codebook_host
    from oracle import tq_oracle as orc
    try:
        from oracle import c_oracle
        clib = c_oracle.load()
    except Exception:
        clib = None
    tables = {b: get_codebook_host(D, b) for b in (1, 2, 3, 4)}
    caches = []
    for li in range(layers):
        rs = np.random.RandomState(seed0 + li)
        k = (rs.randn(1, HKV, CTX, D).astype(np.float32) * np.exp(0.5 * rs.randn(1, HKV, CTX, 1)).astype(np.float32)).astype(np.float16)
        v = (rs.randn(1, HKV, CTX, D).astype(np.float32) * np.exp(0.5 * rs.randn(1, HKV, CTX, 1)).astype(np.float32)).astype(np.float16)
        c = orc.KVCacheOracle(D, tables, 4, 2, RW, fp16_sink_size=SINK)
        if clib is not None:
            c_oracle.use_c_kernels(c, clib)
        c.update_and_fetch(k, v)
        caches.append(c)
    rs = np.random.RandomState(seed0 + 999)
    q = (rs.randn(1, HQ, 1, D) / np.sqrt(D)).astype(np.float16)
    kn = (rs.randn(1, HKV, 1, D)).astype(np.float16)
    threads = clib.tqo_threads() if clib is not None else (os.cpu_count() or 1)

    def step():
        out = None
        for c in caches:
            # the recent-token buffer is restored after the step so every step sees the same 32768+1 tokens
            saved = c.fp_len, c.offset
            dk, dv = c.update_and_fetch(kn, kn)
            out = c_oracle.attention(clib, q, dk, dv) if clib is not None else orc.attention(q, dk, dv)
            c.fp_len, c.offset = saved
        return out

    return step, {"kind": "port", "cores": threads,
                  "sample": f"{layers} of {LAYERS} layers per step; per layer: append 1 token, dense float32 reassembly of "
                            f"{CTX + 1} tokens x {HKV} KV heads, float32 GQA attention ({'C/OpenMP' if clib is not None else 'NumPy'})"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if "WORLD_SIZE" in os.environ:      # torchrun pins OMP_NUM_THREADS to 1; this arm is a CPU job and takes the whole host
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    layers = 1
    step, info = cpu_reference_step_factory(layers)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    gbs = BYTES_PER_LAYER_STEP * layers / dt / 1e9
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "us_per_layer_step": dt / layers * 1e6,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers_per_step": layers, "note": "CPU restatement of the reference's per-step path; MLX and Metal are unavailable on this box"},
        "cpu_baseline": dict(info, value=gbs, unit="GB/s"),
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- the CUDA path ------------------------------------------------------------------------------------------
def build_caches(torch, dev, seq, heads=(0, HKV)):
    """Layer caches of sequence `seq`; `heads` = the KV heads this rank owns (all of them unless heads are split)."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    h0, h1 = heads
    caches, qs = [], []
    for li in range(LAYERS):
        g = torch.Generator(device=dev).manual_seed(1000 + 100 * seq + li)
        scale_k = torch.exp(0.5 * torch.randn(1, HKV, CTX, 1, device=dev, generator=g))
        k = (torch.randn(1, HKV, CTX, D, device=dev, generator=g) * scale_k).half()
        scale_v = torch.exp(0.5 * torch.randn(1, HKV, CTX, 1, device=dev, generator=g))
        v = (torch.randn(1, HKV, CTX, D, device=dev, generator=g) * scale_v).half()
        c = TurboQuantKVCache(head_dim=D, num_kv_heads=h1 - h0, key_bits=4, value_bits=2, residual_window=RW, fp16_sink_size=SINK)
        c.update(k[:, h0:h1].contiguous(), v[:, h0:h1].contiguous())
        assert (c._sink_len, c._compressed_len, c._fp16_len) == (SINK, T_C, RW)
        caches.append(c)
        q = (torch.randn(1, HQ, 1, D, device=dev, generator=g) / D ** 0.5).half()
        qs.append(q[:, h0 * (HQ // HKV):h1 * (HQ // HKV)].contiguous())
        del k, v
    return caches, qs


def bench_quantize(torch, dev, steps, warmup, peak, pool_size=8):
    """Prefill compression throughput: 131072 new tokens x 8 KV heads per layer, chunk_size 4096, residual window
    128 -> the cache drains 31 chunks (126976 tokens) per layer and side, issued as one fused launch each.
    One step = 32 layers (8 distinct fp16 K/V input sets of 0.5 GB each, cycled: every launch reads far more
    than L2 holds).  Two settings: K3/V2 and the mixed-bit K3.5/V3.5."""
    from mlx_turboquant_b200 import kernels
    from mlx_turboquant_b200.codebook import get_codebook
    from mlx_turboquant_b200.rotation import get_rotation_matrix
    rot = get_rotation_matrix(D, 42, dev)
    n_tok = (131072 - RW) // QCHUNK * QCHUNK          # tokens that leave the fp16 buffer: 126976
    g = torch.Generator(device=dev).manual_seed(2000)
    pool = []
    for _ in range(pool_size):
        x = torch.randn(2, 1, HKV, n_tok, D, device=dev, generator=g, dtype=torch.float16)
        x[..., [3, 40, 77, 101]] *= 20.0              # four fixed outlier channels per head
        pool.append(x)
    out = {}
    for name, kb, vb in (("k3_v2", 3, 2), ("k3.5_v3.5", 3.5, 3.5)):
        sides = []
        for bits in (kb, vb):
            hi, lo = kernels.split_bits(bits)
            w_hi, w_lo = kernels.packed_widths(D, hi, lo)
            sides.append(dict(hi=hi, lo=lo, bnd_hi=get_codebook(D, hi, dev)[1], bnd_lo=get_codebook(D, lo, dev)[1] if lo else None,
                              p_hi=torch.empty(1, HKV, n_tok, w_hi, dtype=torch.uint8, device=dev),
                              p_lo=torch.empty(1, HKV, n_tok, w_lo, dtype=torch.uint8, device=dev) if lo else None,
                              norms=torch.empty(1, HKV, n_tok, dtype=torch.float32, device=dev), w=w_hi + w_lo))

        def step():
            for li in range(32):
                x = pool[li % len(pool)]
                for i, s in enumerate(sides):
                    kernels.quantize_pack(x[i], rot, s["bnd_hi"], s["hi"], s["bnd_lo"], s["lo"], out_hi=s["p_hi"],
                                          out_lo=s["p_lo"], out_norms=s["norms"], out_offset=0)
        for _ in range(warmup):
            step()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / steps
        bytes_per_unit = 2 * D * 2 + sides[0]["w"] + 4 + sides[1]["w"] + 4        # per (token, head, layer), K and V
        units = 32 * HKV * n_tok
        gbs = units * bytes_per_unit / (ms * 1e-3) / 1e9
        out[name] = {"mtokens_per_s": n_tok / (ms * 1e-3) / 1e6, "ms_per_step": ms, "tokens_per_step": n_tok,
                     "launches_per_step": 64, "bytes_per_token_head_layer": bytes_per_unit, "hbm_gbs": gbs, "frac_of_peak": gbs / peak}
    del pool
    return out


def bench_quantize_c3(torch, dev, steps, warmup, peak):
    """Prefill compression of one Phi-3.5-mini-shaped layer with the QJL sketch: batch 16 x 32 KV heads x 7936 tokens of
    head_dim 96 leave the fp16 buffer (context 8192, 128 sink, 128 recent), 4-bit keys and 2-bit values, one fused launch per
    side writing codes, norms, sign words and residual norms.  Two distinct input sets (3.1 GB) are cycled."""
    from mlx_turboquant_b200 import kernels
    from mlx_turboquant_b200.codebook import get_codebook
    from mlx_turboquant_b200.qjl import generate_projection_matrix_host
    from mlx_turboquant_b200.rotation import generate_rotation_matrix_host, get_rotation_matrix
    b, h, d, t = 16, 32, 96, 8192 - SINK - RW
    rot = get_rotation_matrix(d, 42, dev)
    prot = torch.from_numpy((generate_projection_matrix_host(d, 32).astype("float64") @ generate_rotation_matrix_host(d, 42).astype("float64").T)
                            .astype("float32")).to(dev)
    g = torch.Generator(device=dev).manual_seed(2100)
    pool = [torch.randn(2, b, h, t, d, device=dev, generator=g, dtype=torch.float16) for _ in range(2)]
    sides = []
    for bits in (4, 2):
        cent, bnd = get_codebook(d, bits, dev)
        sides.append(dict(bits=bits, bnd=bnd, p=torch.empty(b, h, t, d * bits // 8, dtype=torch.uint8, device=dev),
                          n=torch.empty(b, h, t, dtype=torch.float32, device=dev),
                          q=dict(proj_rot=prot, cent_hi=cent, cent_lo=None, bits=torch.empty(b, h, t, dtype=torch.int32, device=dev),
                                 gamma=torch.empty(b, h, t, dtype=torch.float32, device=dev))))

    def step():
        for x in pool:
            for i, sd in enumerate(sides):
                kernels.quantize_pack(x[i], rot, sd["bnd"], sd["bits"], out_hi=sd["p"], out_norms=sd["n"], out_offset=0, qjl=sd["q"])
    for _ in range(warmup):
        step()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / (steps * len(pool))                  # per layer (K and V)
    bytes_per_unit = 2 * d * 2 + (d * 4 // 8 + 4) + (d * 2 // 8 + 4) + 2 * (4 + 4)
    gbs = b * h * t * bytes_per_unit / (ms * 1e-3) / 1e9
    del pool
    return {"workload": "phi35mini_layer_prefill_compress_b16_h32_d96_k4v2_qjl", "ms_per_layer": ms, "rows_per_side": b * h * t,
            "bytes_per_token_head": bytes_per_unit, "hbm_gbs": gbs, "frac_of_peak": gbs / peak, "launches_per_layer": 2}


def bench_c3(torch, dev, steps, warmup, peak):
    """Phi-3.5-mini-shaped layer with the QJL sketch: 32 query = 32 KV heads, head_dim 96, batch 16, context 8192 =
    128 sink + 7936 packed (4-bit keys, 2-bit values, sign sketches) + 128 recent.  One launch = one layer-step;
    four layer caches (1.8 GB) are cycled."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    b, h, d, ctx = 16, 32, 96, 8192
    t_c = ctx - SINK - RW
    bytes_step = b * h * t_c * (d // 2 + 4 + d // 4 + 4 + 2 * (4 + 4)) + b * h * (SINK + RW) * 2 * d * 2 + b * h * d * 4
    caches, qs = [], []
    for li in range(4):
        g = torch.Generator(device=dev).manual_seed(3000 + li)
        k = (torch.randn(b, h, ctx, d, device=dev, generator=g) * torch.exp(0.5 * torch.randn(b, h, ctx, 1, device=dev, generator=g))).half()
        v = (torch.randn(b, h, ctx, d, device=dev, generator=g) * torch.exp(0.5 * torch.randn(b, h, ctx, 1, device=dev, generator=g))).half()
        c = TurboQuantKVCache(head_dim=d, num_kv_heads=h, key_bits=4, value_bits=2, residual_window=RW, fp16_sink_size=SINK,
                              qjl_correction=True)
        c.update(k, v)
        assert (c._sink_len, c._compressed_len, c._fp16_len) == (SINK, t_c, RW)
        caches.append(c)
        qs.append((torch.randn(b, h, 1, d, device=dev, generator=g) / d ** 0.5).half())
        del k, v
    def step():
        for c, q in zip(caches, qs):
            c.attend(q)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize(dev)
    us = e0.elapsed_time(e1) * 1e3 / (steps * len(caches))
    gbs = bytes_step / (us * 1e-6) / 1e9
    import ctypes as C
    from mlx_turboquant_b200 import _lib
    choice = _lib.lib().tq_decode_kernel_choice(C.byref(caches[0]._dargs))
    names = {0: "decode_attn_kernel<96, qjl> (general kernel: unpack to shared memory, ldmatrix)",
             2: "decode_stream_kernel<96, qjl> (persistent grid over the packed tiles of all lanes; stream_query_kernel before it, "
                "stream_merge_kernel after it: three launches per layer-step)"}
    return {"workload": "phi35mini_layer_decode_attn_b16_ctx8192_k4v2_qjl_sink128_rw128", "us_per_layer_step": us,
            "algorithmic_bytes_per_launch": bytes_step, "hbm_gbs": gbs, "frac_of_peak": gbs / peak,
            "kernel": names.get(choice, str(choice))}


def bench_prefill(torch, dev, steps, warmup):
    """One prefill chunk of a Llama-3.1-8B layer straight from packed storage: 4 sequences, 32 query / 8 KV heads,
    head_dim 128, the last 512 tokens of a 16384-token cache (128 sink + packed 4-bit keys / 2-bit values + recent)
    attending causally over all of it.  One launch = one layer-chunk; two layer caches are cycled."""
    from mlx_turboquant_b200 import TurboQuantKVCache
    b, ctx, tq = 4, 16384, 512
    caches, qs = [], []
    for li in range(2):
        g = torch.Generator(device=dev).manual_seed(3500 + li)
        c = TurboQuantKVCache(head_dim=D, num_kv_heads=HKV, key_bits=4, value_bits=2, residual_window=RW, fp16_sink_size=SINK)
        for _ in range(ctx // 4096):
            k = (torch.randn(b, HKV, 4096, D, device=dev, generator=g) * torch.exp(0.5 * torch.randn(b, HKV, 4096, 1, device=dev, generator=g))).half()
            v = (torch.randn(b, HKV, 4096, D, device=dev, generator=g) * torch.exp(0.5 * torch.randn(b, HKV, 4096, 1, device=dev, generator=g))).half()
            c.update(k, v)
        caches.append(c)
        qs.append((torch.randn(b, HQ, tq, D, device=dev, generator=g) / D ** 0.5).half())
        del k, v
    outs = [torch.empty_like(q) for q in qs]

    def step():
        for c, q, o in zip(caches, qs, outs):
            c.attend(q, out=o)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / (steps * len(caches))
    flops = 4.0 * b * HQ * tq * (ctx - tq / 2) * D                  # QK^T and PV over the causal extent
    return {"workload": "llama31_8b_layer_prefill_chunk_b4_ctx16384_tq512_k4v2_sink128_rw128", "ms_per_layer_chunk": ms,
            "tflops": flops / (ms * 1e-3) / 1e12, "query_tokens_per_s": b * tq / (ms * 1e-3),
            "kernel": "prefill_tc_kernel (tcgen05: 128 query rows per CTA, scores and outputs in tensor memory, unpacked tiles as shared-memory operands)"}


def bench_dequantize(torch, dev, steps, warmup, peak):
    """The reference's own read path: dense reassembly of the packed middle (cache.py:276-343) - unpack, centroid lookup,
    inverse rotation, scale - for 16 layers' worth of C1-shaped caches at once (16 x 8 KV heads x 32512 tokens, head_dim 128;
    4-bit keys and 2-bit values -> fp16 rows).  Algorithmic bytes per row: packed codes + norm in, 256 B out."""
    from mlx_turboquant_b200 import kernels
    from mlx_turboquant_b200.codebook import get_codebook
    from mlx_turboquant_b200.rotation import get_rotation_matrix
    rot = get_rotation_matrix(D, 42, dev)
    n_l, t = 16, T_C
    g = torch.Generator(device=dev).manual_seed(2300)
    sides = []
    for bits in (4, 2):
        cent, _ = get_codebook(D, bits, dev)
        sides.append(dict(bits=bits, cent=cent, p=torch.randint(0, 256, (n_l, HKV, t, D * bits // 8), dtype=torch.uint8, device=dev, generator=g),
                          n=torch.rand(n_l, HKV, t, device=dev, generator=g) + 0.5, o=torch.empty(n_l, HKV, t, D, dtype=torch.float16, device=dev)))

    def step():
        for sd in sides:
            kernels.dequantize_rows(sd["p"], None, sd["n"], rot, sd["cent"], sd["bits"], None, 0, D, out=sd["o"])
    for _ in range(warmup):
        step()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / steps
    nbytes = sum(sd["p"].numel() + sd["n"].numel() * 4 + sd["o"].numel() * 2 for sd in sides)
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"workload": "llama31_8b_dense_reassembly_16layers_ctx32768_k4v2_fp16", "ms_per_step": ms, "rows": 2 * n_l * HKV * t,
            "hbm_gbs": gbs, "frac_of_peak": gbs / peak, "kernel": "dequantize_tc_kernel (tcgen05: three split products, accumulators in tensor memory)"}


def bench_head_split(torch, dist, dev, world, rank, steps, warmup):
    """N > 1: the headline workload as ONE sequence whose KV heads are dealt to the GPUs (strong scaling of a single
    sequence), timed three ways in the same process group: every GPU keeps its own heads' outputs (no exchange); the
    kernel's merge step stores its heads into every GPU's buffer and the next layer's kernel waits for the peers' heads in
    its prologue (peer stores + arrival counters, no collective, one wait launch after the last layer); NCCL all-gather
    after every layer.  Per mode: a CUDA graph of the 32 layer calls, device-timed, max over ranks."""
    from mlx_turboquant_b200 import sharding
    plan = sharding.plan_lanes(1, HKV, world, rank, split_heads=True)
    caches, qs = build_caches(torch, dev, 0, (plan.head_begin, plan.head_end))
    g_heads = HQ // HKV
    n_kv = plan.head_end - plan.head_begin
    fused = sharding.FusedGather(1, HQ, D, torch.float16, n_buffers=LAYERS, head_offset=plan.head_begin * g_heads,
                                 n_local_heads=n_kv * g_heads, n_local_kv_heads=n_kv, device=dev)
    gathered = [torch.empty(world, 1, n_kv * g_heads, 1, D, dtype=torch.float16, device=dev) for _ in range(LAYERS)]
    outs = [None] * LAYERS

    def no_gather():
        for i in range(LAYERS):
            outs[i] = caches[i].attend(qs[i])

    def fused_gather():
        for i in range(LAYERS):
            caches[i].attend(qs[i], gather=fused.slot(i), after=fused.arrived(i - 1) if i else None)
        fused.wait(LAYERS - 1)

    def nccl_all_gather():
        for i in range(LAYERS):
            outs[i] = caches[i].attend(qs[i])
            dist.all_gather_into_tensor(gathered[i], outs[i])

    def sync():
        torch.cuda.synchronize(dev)
        dist.barrier()
        torch.cuda.synchronize(dev)

    res = {"workload": WORKLOAD + "_one_sequence_kv_heads_split", "kv_heads_per_gpu": n_kv, "layers_per_step": LAYERS,
           "timing": "CUDA graph of the layer calls, CUDA events, max over ranks"}
    for name, fn in (("no_gather", no_gather), ("fused_gather", fused_gather), ("nccl_all_gather", nccl_all_gather)):
        fn()
        sync()
        launch = "graph"
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
            run = graph.replay
        except Exception:      # a collective that cannot be captured: launched eagerly
            launch, run = "eager", fn
        for _ in range(max(warmup, 3)):
            run()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            run()
        e1.record()
        sync()
        ms = sharding.job_time_ms(e0.elapsed_time(e1) / steps, dev)
        res[name] = {"us_per_layer_step": ms * 1e3 / LAYERS, "launch": launch,
                     "hbm_gbs_all_gpus": LAYERS * BYTES_PER_LAYER_STEP / (ms * 1e-3) / 1e9}
    res["fused_gather"]["over_no_gather_us"] = res["fused_gather"]["us_per_layer_step"] - res["no_gather"]["us_per_layer_step"]
    res["nccl_all_gather"]["over_no_gather_us"] = res["nccl_all_gather"]["us_per_layer_step"] - res["no_gather"]["us_per_layer_step"]
    # the fused path's result is the same bits as the collective's
    want = gathered[LAYERS - 1].reshape(1, HQ, D)
    res["fused_equals_all_gather"] = bool(torch.equal(fused.result(LAYERS - 1), want))
    from mlx_turboquant_b200 import _lib
    res["device_status"] = int(_lib.lib().tq_device_status())
    sync()
    fused.close()
    return res


def run_c4(args):
    """`--workload c4`: end-to-end batched decoding of a random-init Llama-3.1-8B-shaped model (32 layers, hidden 4096,
    32 query / 8 KV heads, head_dim 128, SwiGLU 14336, vocabulary 128256, bf16 weights N(0, 0.02)) through compressed
    caches (4-bit keys, 2-bit values, 128-token sink, 128 recent tokens).  `--c4-batch` sequences in total, dealt evenly
    to the GPUs (every GPU holds the full weights; no collective).  Every sequence has a prompt of `--c4-prompt` random
    token ids, prefilled through the model in `--c4-prefill-chunk`-token pieces (attention of a piece runs straight from
    packed storage); `--c4-prefill synthetic` instead fills the caches with seeded synthetic K/V of the same kind, for
    quick runs.  Then `--steps` tokens are generated greedily; one STEP = one new token for every sequence: embedding,
    32 x (projections, RoPE, cache.decode_step, output projection, SwiGLU), logits, arg-max.  GEMMs and element-wise work
    are torch library calls replayed from CUDA graphs (consumer.GraphedDecoder); the cache calls are this repository's
    kernels.  The timed region is the generation; the prefill is timed separately."""
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")    # caches grow while activations come and go
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from mlx_turboquant_b200 import _lib, apply_turboquant, sharding
    from mlx_turboquant_b200.consumer import GraphedDecoder, LlamaShaped, ModelArgs
    _lib.lib()
    peak, peak_src = peaks()
    assert args.c4_batch % world == 0
    b, prompt, piece = args.c4_batch // world, args.c4_prompt, 4096
    margs = ModelArgs(num_hidden_layers=args.layers)
    model = LlamaShaped(margs, dtype=torch.bfloat16, device=dev, seed=0)
    apply_turboquant(model, key_bits=4, value_bits=2, residual_window=RW, fp16_sink_size=SINK, auto_detect_outliers=False)
    caches = model.make_cache()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    e0.record()
    if args.c4_prefill == "model":
        ids = torch.randint(0, margs.vocab_size, (b, prompt), device=dev, generator=torch.Generator(device=dev).manual_seed(4000 + rank))
        logits = None
        for s0 in range(0, prompt, args.c4_prefill_chunk):
            logits = model(ids[:, s0:s0 + args.c4_prefill_chunk], cache=caches, packed=True, last_only=True)
        tok = logits[:, -1].argmax(-1, keepdim=True)
        del ids, logits
    else:
        for li, c in enumerate(caches):
            g = torch.Generator(device=dev).manual_seed(4000 + 64 * rank + li)
            for s0 in range(0, prompt, piece):
                n = min(piece, prompt - s0)
                kv = []
                for _ in range(2):
                    x = torch.randn(b, HKV, n, D, device=dev, generator=g, dtype=torch.bfloat16)
                    kv.append(x * torch.exp(0.5 * torch.randn(b, HKV, n, 1, device=dev, generator=g)).to(torch.bfloat16))
                c.update(kv[0], kv[1])
            del kv, x
        tok = torch.randint(0, margs.vocab_size, (b, 1), device=dev, generator=torch.Generator(device=dev).manual_seed(5000 + rank))
    e1.record()
    torch.cuda.synchronize(dev)
    prefill_s = e0.elapsed_time(e1) * 1e-3
    torch.cuda.empty_cache()

    if args.no_graph:
        class _Eager:
            tok = None

            def step(self):
                self.tok = model(self.tok, cache=caches, packed=True)[:, -1].argmax(-1, keepdim=True)
        dec = _Eager()
        dec.tok = tok
    else:
        dec = GraphedDecoder(model, caches, tok)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        dec.step()
    barrier()
    ctx0 = caches[0].offset
    with ClockSampler(local) as clk:
        e0.record()
        for _ in range(args.steps):
            dec.step()
        e1.record()
        barrier()
    ms_step = sharding.job_time_ms(e0.elapsed_time(e1) / args.steps, dev)
    prefill_s = sharding.job_time_ms(prefill_s, dev)

    # the attention share: the same caches, `attend` alone (one launch per layer)
    c0 = caches[0]
    q = (torch.randn(b, HQ, 1, D, device=dev) / D ** 0.5).to(torch.bfloat16)
    for c in caches:
        c.attend(q)
    torch.cuda.synchronize(dev)
    e0.record()
    reps = 3
    for _ in range(reps):
        for c in caches:
            c.attend(q)
    e1.record()
    torch.cuda.synchronize(dev)
    attn_us = e0.elapsed_time(e1) * 1e3 / (reps * len(caches))
    attn_bytes = (b * HKV * c0._compressed_len * (D // 2 + 4 + D // 4 + 4) + b * HKV * (c0._sink_len + c0._fp16_len) * 2 * D * 2
                  + b * HQ * D * 4)
    attn_gbs = attn_bytes / (attn_us * 1e-6) / 1e9
    import ctypes as C
    from mlx_turboquant_b200 import _lib
    choice = _lib.lib().tq_decode_kernel_choice(C.byref(c0._dargs))     # 2: streaming kernel = query + persistent grid + merge launches
    launches_per_call = 3 if choice == 2 else 1
    attn_kernel = {0: "decode_attn_kernel", 1: "decode_direct_kernel", 2: "stream_query_kernel + decode_stream_kernel + stream_merge_kernel"}.get(choice, str(choice))
    weight_bytes = sum(p.numel() * p.element_size() for p in model.parameters()) - model.embed_tokens.weight.numel() * 2
    floor_ms = (attn_bytes * args.layers + weight_bytes) / (peak * 1e9) * 1e3
    line = {
        "metric": "e2e_decode_tokens_per_s", "value": args.c4_batch * 1e3 / ms_step, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 weights and activations; attention f32 accumulate over packed 4-bit keys / 2-bit values",
        "data": "synthetic",
        "config": {"workload": "llama31_8b_shaped_batched_decode_k4v2_sink128_rw128", "layers": args.layers, "batch_total": args.c4_batch,
                   "batch_per_gpu": b, "context_at_start": ctx0, "context_at_end": caches[0].offset,
                   "prompt": ("random token ids prefilled through the model in %d-token pieces" % args.c4_prefill_chunk) if args.c4_prefill == "model"
                   else "cache contents from seeded synthetic K/V (no prefill pass)",
                   "decode_step": "eager" if args.no_graph else "library part replayed from CUDA graphs, cache calls eager",
                   "l2_policy": "inputs larger than L2",
                   "sharding": "sequences dealt to the GPUs, full weights on each, no collective"},
        "gpu_launches": args.layers * args.steps * launches_per_call,
        "clocks": clk.summary(),
        "prefill": {"seconds": prefill_s, "tokens_per_s": args.c4_batch * prompt / prefill_s, "mode": args.c4_prefill},
        "attention": {"us_per_layer_step": attn_us, "algorithmic_bytes_per_launch": attn_bytes, "hbm_gbs": attn_gbs, "frac_of_peak": attn_gbs / peak,
                      "peak": peak, "peak_source": peak_src, "share_of_step": attn_us * args.layers / (ms_step * 1e3), "kernel": attn_kernel},
        "hbm_floor_ms_per_step": floor_ms, "step_over_floor": ms_step / floor_ms,
        "weight_read_floor_ms_per_step": weight_bytes / (peak * 1e9) * 1e3,
        "cache_bytes_per_gpu": sum(c.nbytes for c in caches), "weight_bytes_read_per_step": weight_bytes,
    }
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_b200(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    import __graft_entry__ as ge
    from mlx_turboquant_b200 import _lib, sharding
    if not _lib.LIB_PATH.exists() and rank == 0:
        ge.build()
    if world > 1:
        dist.barrier()
    _lib.lib()
    peak, peak_src = peaks()

    global LAYERS
    LAYERS = args.layers
    if args.split_heads and world > 1:
        # strong scaling of ONE sequence: its KV heads dealt to the ranks; per layer the (1, H_q / world, 1, D) outputs
        # are all-gathered (the only collective on the path), unless --no-gather
        plan = sharding.plan_lanes(1, HKV, world, rank, split_heads=True)
        caches, qs = build_caches(torch, dev, 0, (plan.head_begin, plan.head_end))
        n_seq = 1
    else:
        # weak scaling: `world` independent sequences, dealt one per rank; no rank reads another rank's lanes
        plan = sharding.plan_lanes(world, HKV, world, rank, split_heads=False)
        assert (plan.seq_end - plan.seq_begin, plan.head_end - plan.head_begin) == (1, HKV)
        caches, qs = build_caches(torch, dev, plan.seq_begin)
        n_seq = world
    split = args.split_heads and world > 1
    if split:
        args.no_e2e = True            # the host-buffer leg is defined for whole sequences per GPU
    torch.cuda.synchronize(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident throughput: CUDA graph of one 32-layer step -------------------------------------
    outs = [None] * LAYERS

    fused = None
    if split and args.fused_gather:
        # every rank's result buffers (one slot per layer) mapped into every rank: the kernel's merge step stores this rank's
        # heads into all of them and the consumer waits on an arrival counter - no collective on the path
        g_heads = HQ // HKV
        fused = sharding.FusedGather(1, HQ, D, torch.float16, n_buffers=LAYERS, head_offset=plan.head_begin * g_heads,
                                     n_local_heads=(plan.head_end - plan.head_begin) * g_heads,
                                     n_local_kv_heads=plan.head_end - plan.head_begin, device=dev)

    def layer_pass():
        for i in range(LAYERS):
            if fused is not None:
                caches[i].attend(qs[i], gather=fused.slot(i))
                fused.wait(i)
                outs[i] = fused.result(i)
                continue
            outs[i] = caches[i].attend(qs[i])
            if split and not args.no_gather:
                outs[i] = sharding.gather_heads(outs[i])
    layer_pass()                      # allocates the workspace before capture
    torch.cuda.synchronize(dev)
    if args.no_graph or (split and fused is None):        # collectives are launched eagerly
        class _Eager:
            replay = staticmethod(layer_pass)
        graph = _Eager()
    else:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            layer_pass()
    launches_per_step = LAYERS          # one fused kernel per layer call
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    barrier()
    with ClockSampler(local) as clk:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # keep the timed region long enough for clock samples
        reps = args.steps
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        barrier()
        ms_step = e0.elapsed_time(e1) / reps
        # a few more replays so the sampler sees the loaded clock; a fixed count when the step holds collectives
        # (every rank must issue the same number of them), wall-clock bounded otherwise
        if split and not args.no_gather:
            for _ in range(200):
                graph.replay()
        else:
            t_end = time.time() + (0.0 if args.no_graph else 0.6)
            while time.time() < t_end:
                graph.replay()
        torch.cuda.synchronize(dev)
    ms_step = sharding.job_time_ms(ms_step, dev)
    value = n_seq * LAYERS * BYTES_PER_LAYER_STEP / (ms_step * 1e-3) / 1e9

    # ---- end to end through the public API with host buffers -----------------------------------------------
    # one pinned staging buffer holds the step's query, key and value heads of all layers: one host -> device copy per step;
    # the results of all layers leave in one device -> host copy at the end of the step
    hx = torch.randn(LAYERS, 1, HQ + 2 * HKV, 1, D).half().pin_memory()
    hout = torch.empty(LAYERS, 1, HQ, 1, D, dtype=torch.float16).pin_memory()
    xdev, odev = torch.empty_like(hx, device=dev), torch.empty_like(hout, device=dev)
    xq = [xdev[i][:, :HQ] for i in range(LAYERS)]
    xk = [xdev[i][:, HQ:HQ + HKV] for i in range(LAYERS)]
    xv = [xdev[i][:, HQ + HKV:] for i in range(LAYERS)]
    xo = [odev[i] for i in range(LAYERS)]
    e2e_caches, _ = (caches, None)

    def e2e_step():
        xdev.copy_(hx, non_blocking=True)
        for i in range(LAYERS):
            e2e_caches[i].decode_step(xq[i], xk[i], xv[i], out=xo[i])
        hout.copy_(odev, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
    e2e_steps = min(args.steps, 20)
    for _ in range(0 if args.no_e2e else 3):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(0 if args.no_e2e else e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = sharding.job_time_ms(e0.elapsed_time(e1) / e2e_steps, dev)
    e2e_gbs = None if args.no_e2e else n_seq * LAYERS * BYTES_PER_LAYER_STEP / (e2e_ms * 1e-3) / 1e9

    line = {
        "metric": "decode_attn_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "us_per_layer_step": ms_step * 1e3 / LAYERS,
        "higher_is_better": True, "scaling": "strong" if split else "weak", "vs_baseline": None, "dtype": "f32 accumulate, f16 operands",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers_per_step": LAYERS, "q_heads": HQ, "kv_heads": HKV, "head_dim": D,
                   "batch_per_gpu": 1, "context": CTX, "l2_policy": "inputs larger than L2: 32 distinct layer caches, 0.9 GB per step",
                   "sharding": ("one sequence, KV heads split over the GPUs, " + ("no gather" if args.no_gather else "outputs stored into every GPU's buffer by the kernel's merge step (peer stores + arrival counters)"
                                                                                  if args.fused_gather else "outputs all-gathered per layer (NCCL)"))
                   if split else "independent sequences per GPU, no collective"},
        "e2e": {"value": e2e_gbs, "unit": "GB/s", "ms_per_step": e2e_ms, "us_per_layer_step": e2e_ms * 1e3 / LAYERS,
                "h2d_bytes_per_step": LAYERS * (HQ * D * 2 + 2 * HKV * D * 2), "d2h_bytes_per_step": LAYERS * HQ * D * 2,
                "path": "per step: one pinned-host -> device copy of all layers' q/k/v, TurboQuantKVCache.decode_step per layer (append + attention, one launch), one device -> pinned-host copy of all layers' results"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clk.summary(),
        "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s", "frac": value / world / peak,
                     "peak_source": peak_src, "frac_of_nominal_8tbs": value / world / 8000.0,
                     "traffic": ncu_traffic_bytes(), "traffic_unit": "bytes per launch (ncu, one capture)", "traffic_source": DECODE_PROFILE,
                     "kernel": "decode_direct_kernel<4> (one launch per layer: query rotation on the tensor cores, attention over packed and fp16 tokens, last-arrival merge)",
                     "algorithmic_bytes_per_launch": BYTES_PER_LAYER_STEP},
    }
    if rank == 0 and world == 1 and not args.no_secondary:
        legs = set(args.legs.split(","))
        line["secondary"] = {"metric": "quantize_pack_mtokens_per_s", "unit": "Mtokens/s (token = position x 8 KV heads x 32 layers)", "chunk_tokens": QCHUNK}
        if "quantize" in legs:
            line["secondary"].update(bench_quantize(torch, dev, 3, 3, peak, args.quantize_pool))
        if "compress_c3" in legs:
            line["secondary"]["compress_qjl_d96_b16"] = bench_quantize_c3(torch, dev, 3, 2, peak)
        if "decode_c3" in legs:
            line["secondary"]["decode_qjl_d96_b16"] = bench_c3(torch, dev, 5, 3, peak)
        if "dequantize" in legs:
            line["secondary"]["dequantize_k4v2"] = bench_dequantize(torch, dev, 3, 2, peak)
        if "prefill" in legs:
            line["secondary"]["prefill_chunk_attn"] = bench_prefill(torch, dev, 3, 2)
    if world > 1 and not split and not args.no_secondary and HKV % world == 0:
        hs = bench_head_split(torch, dist, dev, world, rank, args.steps, args.warmup)
        line["secondary"] = {"head_split": hs}
    if rank == 0 and world == 1 and not args.no_cpu:
        step, info = cpu_reference_step_factory(1)
        step()
        t0 = time.perf_counter()
        n = 3
        for _ in range(n):
            step()
        dt = (time.perf_counter() - t0) / n
        line["cpu_baseline"] = dict(info, value=BYTES_PER_LAYER_STEP / dt / 1e9, unit="GB/s", us_per_layer_step=dt * 1e6)
    if rank == 0:
        print(json.dumps(line))
    if fused is not None:
        line_status = _lib.lib().tq_device_status()
        if line_status:
            print(f"rank {rank}: device status {line_status} (a bounded wait ran out)", file=sys.stderr)
        torch.cuda.synchronize(dev)
        dist.barrier()
        fused.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=("b200", "reference"))
    ap.add_argument("--layers", type=int, default=32, help="distinct layer caches per step (32 = the model; fewer for profiling)")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph (for profilers)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--quantize-pool", type=int, default=8, help="distinct 0.5 GB fp16 K/V input sets the quantize leg cycles through")
    ap.add_argument("--split-heads", action="store_true", help="N > 1: shard ONE sequence by KV head (strong scaling) instead of one sequence per GPU")
    ap.add_argument("--no-gather", action="store_true", help="with --split-heads: leave every GPU with its own heads' outputs")
    ap.add_argument("--fused-gather", action="store_true", help="with --split-heads: the decode kernel stores its heads into every GPU's "
                    "result buffer (peer-mapped memory) instead of an NCCL all-gather")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary legs")
    ap.add_argument("--legs", default="quantize,compress_c3,decode_c3,dequantize,prefill", help="which secondary legs run (comma list; profilers "
                    "capture one kernel at a time with little else on the device)")
    ap.add_argument("--workload", default="c1", choices=("c1", "c4"), help="c1: the headline layer-decode benchmark; c4: end-to-end "
                    "batched decoding of a Llama-3.1-8B-shaped model through compressed caches (about 75 GB on the device at the defaults)")
    ap.add_argument("--c4-batch", type=int, default=64, help="c4: sequences in total over all GPUs")
    ap.add_argument("--c4-prompt", type=int, default=32768, help="c4: context length every sequence starts from")
    ap.add_argument("--c4-prefill", default="model", choices=("model", "synthetic"), help="c4: prefill the prompt through the model, "
                    "or fill the caches with synthetic K/V")
    ap.add_argument("--c4-prefill-chunk", type=int, default=512, help="c4: prompt tokens per prefill call")
    ap.add_argument("--no-stream", action="store_true", help="never take the persistent streaming decode kernel (profiling the other two kernels "
                    "on the shapes it would take)")
    args = ap.parse_args()
    if args.no_stream and args.impl != "reference":
        from mlx_turboquant_b200.kernels import set_tuning
        set_tuning("decode_stream", 0)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "c4":
        run_c4(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
