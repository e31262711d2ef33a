#!/usr/bin/env python
"""Benchmark of the Hy3 attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1): decode attention with an INT8 KV cache, batch 1, 80 independent layer caches of
32768 positions each, 64 query heads over 8 KV heads, head_dim 128.  One STEP = one new token:
for each of the 80 layers ONE launch normalises, rotates, quantises and stores the token (fused
QK-RMSNorm + RoPE + quantise/append) and attends over all positions with the split-KV decode
kernel.  The 80 launches of a step are replayed as one CUDA graph; lengths live in device memory.
Metric: decode attention KV GB/s = algorithmic KV bytes read per step (ntok x 2080 B per layer,
i.e. codes + fp16 scales of K and V) / time.  Synthetic seeded N(0,1) data, random "weights".
The block of K timed steps is repeated (--blocks, default 10); value / ms_per_step are the median
block, min and max are printed beside them.

N>1 (weak scaling): every rank holds 32768 positions per layer of ONE sequence of 32768*N tokens
(sequence sharding); per layer ONE launch per rank: the decode kernel's epilogue stores the rank's {m,l,acc}
records into every rank's gather buffer over NVLink peer memory, waits for the others' and folds them
(--nccl-exchange: partial records, NCCL all-gather, merge kernel instead).  After the timed region every rank also
runs the NCCL variant on three layers and the line carries the comparison ("parity").

Secondary objects in the same JSON line:
  N=1: "prefill" / "prefill_int8" / "prefill_multiturn" (configs[2], tensor roofline), "decode_fp16" (the headline
       workload with an FP16 cache, 16 layer caches), "ragged_batch" (configs[4] on one GPU), "long_context_int4" and "long_context_int4_1m" (configs[3] on one GPU), "reference_gpu_kernel" (the
       reference's own CUDA decode kernels on the same GPU, context only);
  N>1: "long_context_int4_sharded" (configs[3]: ONE sequence of 262144 and of 1048576 positions split by token range,
       strong scaling, with rank 0's unsharded time of the same total beside it) and "ragged_kv_head_sharded"
       (configs[4] split by KV head, no collective).

--impl reference: the reference engine's own CPU attention() (hy3.c:617-652, compiled from the
reference sources into oracle/_ref; falls back to the C restatement in oracle/) on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_LAYERS, NTOK, H, G, D = 80, 32768, 64, 8, 128
INT8_BYTES_PER_TOKEN_LAYER = 2 * G * (D + 2)       # 2080: K and V, 8 heads x (128 codes + fp16 scale)
BYTES_PER_TOKEN = {"int8": 2080, "int4": 1056, "fp16": 4096}
SEED = 0x4859335F53454544
METRIC, UNIT = "decode_attn_kv_GBps", "GB/s"
WORKLOAD = ("configs[1]: INT8-KV decode attention, batch 1, 80 independent layer caches x 32768 positions, "
            "64 Q / 8 KV heads, head_dim 128, one token appended per layer per step (fused norm+RoPE+quantise), 1 GPU")
KERNEL_NAME = {"int8": "hy3a_decode_umma_kernel (INT8: scores on mma.sync s8, P.V on tcgen05.mma kind::i8)",
               "int4": "hy3a_decode_kernel<int4>", "fp16": "hy3a_decode_kernel<fp16>"}
COMPUTE = {"int8": "scores: int8 mma.sync with two-digit queries; P.V: tcgen05.mma kind::i8 with two-digit weights, TMEM accumulators; fp32 softmax",
           "int4": "int8 mma.sync scores, fp16 mma.sync P.V, fp32 accumulate/softmax",
           "fp16": "fp16 mma.sync, fp32 accumulate/softmax"}


def _peaks_file():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    return json.load(open(p)) if os.path.exists(p) else None


def hbm_peak():
    m = _peaks_file()
    if m:
        return m["hbm_gbs"], "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s)"


def tensor_peak():
    m = _peaks_file()
    if m:
        return m["bf16_tflops"], "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return 1590.0, "fallback (1.59 PFLOP/s)"


def hbm_roofline(kernel, gbs):
    peak, src = hbm_peak()
    return {"bound": "hbm", "kernel": kernel, "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
            "frac_of_nominal_8TBs": gbs / 8000.0, "peak_source": src}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) >= 9:
                for nme, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(nme)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------- CPU arms
class CpuSample:
    """A bounded sample of the workload on the reference CPU attention: K/V are generated and loaded ONCE; run() is one
    pass over the sample.  The value is quoted in GB/s of INT8-equivalent KV bytes (tokens x 2080 B), the unit of work
    of the GPU arm."""

    def __init__(self, all_threads):
        import numpy as np
        import oracle
        cores = os.cpu_count() or 1
        rng = np.random.default_rng(1)
        self.host_cores = cores
        if oracle.ref_cpu is not None:
            ntok = 4096           # hy3.c:628-629 caps the reference at 4096 keys; longer inputs are silently truncated
            nl = max(1, min(N_LAYERS, cores // 8 * 2)) if all_threads else 1
            K = rng.standard_normal((ntok, G, D)).astype(np.float32)
            V = rng.standard_normal((ntok, G, D)).astype(np.float32)
            for l in range(nl):
                oracle.ref_cpu.load_layer(K, V, l)
            q = rng.standard_normal((nl, H, D)).astype(np.float32)
            if all_threads:
                # the team size is set explicitly from the host's core count: it must not depend on OMP_NUM_THREADS of the
                # launching shell (torchrun exports OMP_NUM_THREADS=1 to its workers)
                team = oracle.ref_cpu.set_threads(cores)
                self.fn = lambda: oracle.ref_cpu.attention_layers(q, ntok)
                threads = min(team, nl * 8)
            else:
                self.fn = lambda: oracle.ref_cpu.attention(q[0], ntok, 0)
                threads = 1
            self.kind = "reference"
            self.sample = ("hy3.c attention() as shipped (-O3 -ffast-math), fp32 KV, %d layer(s) x first %d of 32768 positions "
                           "(the reference caps at 4096 keys), %d thread(s)" % (nl, ntok, threads))
        else:
            ntok, nl, threads, self.kind = NTOK, 1, 1, "port"
            K = rng.standard_normal((ntok, G, D)).astype(np.float32)
            V = rng.standard_normal((ntok, G, D)).astype(np.float32)
            q = rng.standard_normal((1, H, D)).astype(np.float32)
            self.fn = lambda: oracle.attention(q[0], K, V)
            self.sample = "C restatement of hy3.c attention(), fp32 KV, 1 layer x 32768 positions, 1 thread"
        self.ntok, self.nl, self.threads = ntok, nl, threads

    def run(self):
        t0 = time.perf_counter()
        self.fn()
        return time.perf_counter() - t0

    def gbs(self, seconds):
        return self.nl * self.ntok * INT8_BYTES_PER_TOKEN_LAYER / seconds / 1e9

    def describe(self, seconds):
        return {"value": self.gbs(seconds), "unit": UNIT, "cores": self.threads, "kind": self.kind, "sample": self.sample,
                "ms_per_call": seconds * 1e3, "host_cores": self.host_cores,
                "fp32_kv_GBps": self.nl * self.ntok * 2 * G * D * 4 / seconds / 1e9, "layers": self.nl, "ntok": self.ntok}


def cpu_attention_sample(seconds, all_threads):
    """Median time of repeated passes over the bounded sample for about `seconds` (at least 3 passes)."""
    s = CpuSample(all_threads)
    s.run()
    times = []
    t_end = time.perf_counter() + seconds
    while time.perf_counter() < t_end or len(times) < 3:
        times.append(s.run())
    return s.describe(statistics.median(times))


def run_reference(args):
    """The reference arm: one step = one pass of the bounded sample on all host threads; W warm-up, K timed."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    s = CpuSample(True)
    for _ in range(args.warmup):
        s.run()
    times = [s.run() for _ in range(args.steps)]
    per_step = sum(times) / len(times)
    value = s.gbs(per_step)
    cb = {k: v for k, v in s.describe(per_step).items() if k in ("unit", "cores", "kind", "sample", "host_cores")}
    cb["value"] = value
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": per_step * 1e3, "ms_per_step_min": min(times) * 1e3, "ms_per_step_max": max(times) * 1e3,
                      "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD},
                      "cpu_baseline": cb, "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "gpu_launches": 0}))


# ------------------------------------------------------------------------------------- GPU arm: secondary workloads
def ragged_lengths():
    import numpy as np
    rng = np.random.default_rng(SEED)
    return [int(1024 + rng.integers(0, 64513)) for _ in range(64)]


def yarn4_table():
    import numpy as np
    inv = (1.0 / (11158840.0 ** (np.arange(64) / 64.0))).astype(np.float32)
    return inv / 4.0, 1.0 + 0.1 * np.log(4.0)      # every frequency interpolated: the speed does not depend on the blend


def timed_decode_steps(torch, dev, ctx, lens, steps, warm, enqueue, sync_all=None, rope_pos=None):
    """`warm` + `steps` single launches, each timed with CUDA events on the launching stream; returns the per-launch ms."""
    B = len(lens)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    t, times = 0, []
    for i in range(warm + steps):
        ctx.batch_set(list(range(B)), [n + t for n in lens], None if rope_pos is None else [p + t for p in rope_pos])
        if sync_all:
            sync_all()
        ev[0].record(torch.cuda.current_stream(dev))
        enqueue()
        ev[1].record(torch.cuda.current_stream(dev))
        ev[1].synchronize()
        if i >= warm:
            times.append(ev[0].elapsed_time(ev[1]))
        t += 1
    return times


def batch_section(torch, dev, kind, ntok=262144):
    """Secondary decode workloads on one GPU, device-timed fused steps:
    'ragged'  -- configs[4]: 64 sequences, lengths 1024 + (rng % 64513) (seeded), INT8 KV, one token per sequence per
                 step (all 8 KV heads on this GPU), one layer per step (4.2 GB per launch);
    'long'    -- configs[3]: batch 1, INT4 KV, `ntok` positions, YaRN factor 4 (attn_factor on q and k); a step is the
                 token's pass over 4 layer caches, launched back to back as a model's layers are."""
    from hy3_b200 import Hy3Attn
    if kind == "ragged":
        kv, lens, layers = "int8", ragged_lengths(), 1
        what = "configs[4]: 64 sequences, lengths uniform in [1024, 65536] (seeded), INT8 KV, 1 layer, all 8 KV heads on one GPU"
    else:
        kv, lens, layers = "int4", [ntok], 4
        what = "configs[3]: batch 1, INT4 KV, %d positions, YaRN factor 4, 4 layer caches per step, unsharded" % ntok
    B = len(lens)
    steps, warm = 20, 4
    ctx = Hy3Attn(kv_dtype=kv, n_layers=layers, max_seqs=B, max_batch=B, max_tokens=sum(lens) + (steps + warm + 129) * B,
                  max_tokens_per_seq=max(lens) + steps + warm + 129, device=dev.index)
    if kind == "long":
        ctx.set_rope(*yarn4_table())
    for l in range(layers):
        for i, n in enumerate(lens):
            ctx.fill_random(l, i, 0, n, SEED + i + 1000 * l)
    q = torch.randn((B, H, D), device=dev)
    k = torch.randn((B, G, D), device=dev)
    v = torch.randn((B, G, D), device=dev)
    out = torch.zeros((layers, B, H, D), device=dev)

    def step():
        for l in range(layers):
            ctx.decode_step(l, q, k, v, out=out[l])
    times = [t / layers for t in timed_decode_steps(torch, dev, ctx, lens, steps, warm, step)]
    ctx.sync()
    ctx.close()
    ms = statistics.median(times)
    nbytes = (sum(lens) + B * (warm + steps // 2)) * BYTES_PER_TOKEN[kv]
    gbs = nbytes / ms / 1e6
    return {"metric": METRIC, "value": gbs, "unit": UNIT, "workload": what, "ms_per_launch": ms, "ms_per_launch_min": min(times),
            "ms_per_launch_max": max(times), "launches_per_step": layers, "algorithmic_bytes_per_launch": nbytes,
            "l2": "%.2f GB streamed per step, far beyond L2" % (layers * nbytes / 1e9), "roofline": hbm_roofline(KERNEL_NAME[kv], gbs)}


def decode_cache_type_section(torch, dev, kv, layers=16, ntok=NTOK):
    """The headline workload with another cache type (FP16 KV): batch 1, `layers` independent layer caches x `ntok`
    positions, a step = one fused launch per layer, replayed as one CUDA graph; blocks of 20 steps, median."""
    from hy3_b200 import Hy3Attn
    steps, warm, blocks = 20, 3, 5
    ctx = Hy3Attn(kv_dtype=kv, n_layers=layers, max_batch=1, max_tokens=ntok + steps + 300, device=dev.index)
    stream = torch.cuda.Stream(device=dev)
    ctx.set_stream(stream)
    for l in range(layers):
        ctx.fill_random(l, 0, 0, ntok, SEED + l)
    with torch.cuda.stream(stream):
        q = torch.randn((layers, 1, H, D), device=dev)
        k = torch.randn((layers, 1, G, D), device=dev)
        v = torch.randn((layers, 1, G, D), device=dev)
        out = torch.zeros((layers, 1, H, D), device=dev)

    def step():
        for l in range(layers):
            ctx.decode_step(l, q[l], k[l], v[l], out=out[l])
    ctx.batch_set([0], [ntok])
    with torch.cuda.stream(stream):
        step()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    ctx.batch_set([0], [ntok + 1])
    with torch.cuda.graph(graph, stream=stream):
        step()
    stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    per_launch = []
    for b in range(blocks + 1):
        e0.record(stream)
        for s in range(steps if b else warm):
            ctx.batch_set([0], [ntok + 2 + s])
            with torch.cuda.stream(stream):
                graph.replay()
        e1.record(stream)
        stream.synchronize()
        if b:
            per_launch.append(e0.elapsed_time(e1) / (steps * layers))
    ctx.sync()
    del graph
    ctx.close()
    ms = statistics.median(per_launch)
    nbytes = (ntok + 2 + steps // 2) * BYTES_PER_TOKEN[kv]
    gbs = nbytes / ms / 1e6
    return {"metric": METRIC, "value": gbs, "unit": UNIT,
            "workload": "%s-KV decode attention, batch 1, %d independent layer caches x %d positions, one fused launch per layer, graph of %d launches" % (kv, layers, ntok, layers),
            "us_per_launch": ms * 1e3, "us_per_launch_min": min(per_launch) * 1e3, "us_per_launch_max": max(per_launch) * 1e3,
            "algorithmic_bytes_per_launch": nbytes, "l2": "%.2f GB streamed per step, far beyond L2" % (layers * nbytes / 1e9),
            "roofline": hbm_roofline(KERNEL_NAME[kv], gbs)}


def prefill_section(torch, dev, kv="fp16", prompt=8192, chunk=512, prefix=0):
    """Chunked causal prefill attention (configs[2]): `prompt` tokens in `chunk`-token chunks on top of a cached prefix of
    `prefix` tokens, 64 Q / 8 KV heads, one layer.  TFLOP/s = 4*128*64*sum(pos+1) over the NEW rows / device time of the
    attention calls (conversion of pages not yet in the fp16 operand mirror, if any, + tcgen05 kernel); the fused append
    -- which also writes the chunk's rows through into the mirror -- is timed separately, and chunk_path_TFLOPs divides
    by the sum of both.  cold_ms: the first ingest of the new rows on the fresh context, before any warm-up."""
    from hy3_b200 import Hy3Attn
    total = prefix + prompt
    ctx = Hy3Attn(kv_dtype=kv, n_layers=1, max_batch=chunk, max_tokens=total + 256, device=dev.index)
    q = torch.randn((total, H, D), device=dev)
    k = torch.randn((total, G, D), device=dev)
    v = torch.randn((total, G, D), device=dev)
    q16 = torch.empty((chunk, H, D), dtype=torch.float16, device=dev)
    out = torch.zeros((chunk, H, D), device=dev)

    def ingest(b0, b1, timed):
        att, app = [], []
        for b in range(b0, b1, chunk):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ctx.batch_set([0] * chunk, list(range(b, b + chunk)))
            ev[0].record()
            ctx.append(0, q[b:b + chunk], k[b:b + chunk], v[b:b + chunk], q_out=False, q_out16=q16)
            ev[1].record()
            ctx.prefill(0, 0, b, q16, out=out)
            ev[2].record()
            att.append((ev[1], ev[2])); app.append((ev[0], ev[1]))
        torch.cuda.synchronize()
        return (sum(a.elapsed_time(b) for a, b in att), sum(a.elapsed_time(b) for a, b in app)) if timed else None

    def run():
        if prefix:
            ctx.seq_release(0, prefix)          # back to the cached prefix (prefix reuse: hy3.c:1514)
        return ingest(prefix, total, True)

    if prefix:
        ingest(0, prefix, False)
    cold = run()
    for _ in range(3):
        run()
    att_ms, app_ms = min(run() for _ in range(5))
    ctx.sync()
    launches = ctx.launches
    ctx.close()
    pairs = sum(prefix + c * chunk + i + 1 for c in range(prompt // chunk) for i in range(chunk))
    flops = 4.0 * D * H * pairs
    peak, src = tensor_peak()
    tf = flops / att_ms / 1e9
    return {"metric": "prefill_attn_TFLOPs", "value": tf, "unit": "TFLOP/s",
            "workload": "configs[2]: %d new tokens in %d-token chunks%s, %s KV, 1 layer" % (
                prompt, chunk, (" after a cached prefix of %d tokens" % prefix) if prefix else "", kv),
            "attention_ms_per_layer": att_ms, "append_ms_per_layer": app_ms, "algorithmic_tflop_per_layer": flops / 1e12,
            "chunk_path_TFLOPs": flops / (att_ms + app_ms) / 1e9, "cold_ms": cold[0] + cold[1],
            "roofline": {"bound": "tensor", "kernel": "hy3a_prefill_kernel", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                         "frac_of_nominal_2250": tf / 2250.0, "peak_source": src},
            "gpu_launches_total": launches}


def reference_gpu_kernel_section():
    """The reference's own CUDA decode kernels (hy3_gpu.cu:183-247, compiled from the reference's sources for plain
    sm_100 into oracle/_ref) on the headline shape: INT8 slots, 32768 keys, the split count the reference picks, caches
    of 16 layers cycled so that launches do not re-read L2.  Context for the published numbers, not the bar."""
    try:
        import oracle
        ref = oracle.ref_gpu()
        if ref is None:
            return {"unavailable": "oracle/_ref/libhy3ref_gpu.so is not built"}
        ms = ref.decode_bench(NTOK, 16, 64)
        gbs = NTOK * INT8_BYTES_PER_TOKEN_LAYER / ms / 1e6
        return {"metric": METRIC, "value": gbs, "unit": UNIT, "us_per_layer": ms * 1e3,
                "workload": "hy3_gpu.cu attention_split_kv_kernel + attention_reduce_kernel, INT8 slots, 32768 keys, 1 layer per launch pair, 16 caches cycled",
                "frac_of_hbm_peak": gbs / hbm_peak()[0]}
    except Exception as e:       # the harness is optional context: never fail the bench line for it
        return {"unavailable": "%s: %s" % (type(e).__name__, e)}


# ------------------------------------------------------------------------------------- GPU arm: multi-GPU secondary workloads
def gather_max(torch, dist, dev, x):
    t = torch.tensor([x], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def long_sharded_section(torch, dist, dev, rank, world, total):
    """configs[3]: ONE sequence of `total` positions, INT4 KV, YaRN factor 4, split by token range
    (hy3_b200.sharding.sequence_range); a step is the token's pass over 4 layer caches; the in-kernel exchange over peer
    memory folds the ranks' records.  Strong scaling: the same total on rank 0 alone is timed right after, in the same
    process."""
    from hy3_b200 import Hy3Attn
    from hy3_b200.sharding import sequence_range
    steps, warm, layers = 20, 4, 4
    t0, t1 = sequence_range(rank, world, total)
    mine = t1 - t0
    owner = rank == world - 1
    ctx = Hy3Attn(kv_dtype="int4", n_layers=layers, max_batch=1, max_tokens=mine + steps + warm + 256, device=dev.index)
    ctx.set_rope(*yarn4_table())
    for l in range(layers):
        ctx.fill_random(l, 0, 0, mine, SEED + 77 * rank + 1000 * l)
    handles = [None] * world
    dist.all_gather_object(handles, ctx.shard_init(rank, world, layers, 1))
    ctx.shard_connect(handles)
    dist.barrier()
    q = torch.randn((1, H, D), device=dev)
    k = torch.randn((1, G, D), device=dev)
    v = torch.randn((1, G, D), device=dev)
    out = torch.zeros((layers, 1, H, D), device=dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    times = []
    for i in range(warm + steps):
        ctx.batch_set([0], [mine + i if owner else mine - 1], [total + i])
        dist.barrier()
        torch.cuda.synchronize()
        ev[0].record(torch.cuda.current_stream(dev))
        for l in range(layers):
            ctx.decode_step_sharded(l, l, q, k if owner else None, v if owner else None, out=out[l])
        ev[1].record(torch.cuda.current_stream(dev))
        ev[1].synchronize()
        ms = gather_max(torch, dist, dev, ev[0].elapsed_time(ev[1])) / layers
        if i >= warm:
            times.append(ms)
    ctx.sync()
    dist.barrier()
    ctx.shard_disconnect()
    ctx.close()
    ms = statistics.median(times)
    nbytes = (total + warm + steps // 2) * BYTES_PER_TOKEN["int4"]
    res = {"positions": total, "ms_per_launch": ms, "ms_per_launch_min": min(times), "ms_per_launch_max": max(times),
           "launches_per_step": layers, "value": nbytes / ms / 1e6, "unit": UNIT, "algorithmic_bytes_per_launch": nbytes}
    # the same total on one GPU (rank 0), for the strong-scaling ratio
    one = None
    if rank == 0:
        one = batch_section(torch, dev, "long", ntok=total)
    dist.barrier()
    if rank == 0:
        res["one_gpu_ms_per_launch"] = one["ms_per_launch"]
        res["one_gpu_value"] = one["value"]
        res["speedup_vs_one_gpu"] = one["ms_per_launch"] / ms
        res["strong_scaling_efficiency"] = one["ms_per_launch"] / ms / world
        res["frac_of_aggregate_hbm_peak"] = res["value"] / (hbm_peak()[0] * world)
    return res


def ragged_head_sharded_section(torch, dist, dev, rank, world):
    """configs[4]: the seeded 64-sequence ragged batch, INT8 KV, split by KV head (hy3_b200.sharding.kv_head_range): rank r
    holds heads [r*8/N, (r+1)*8/N) of every sequence and writes the matching query heads' outputs; no collective."""
    from hy3_b200 import Hy3Attn
    from hy3_b200.sharding import kv_head_range
    lens = ragged_lengths()
    B = len(lens)
    steps, warm = 20, 4
    h0, hc = kv_head_range(rank, world)
    ctx = Hy3Attn(kv_dtype="int8", n_layers=1, kv_head_begin=h0, kv_head_count=hc, max_seqs=B, max_batch=B,
                  max_tokens=sum(lens) + (steps + warm + 129) * B, max_tokens_per_seq=max(lens) + steps + warm + 129, device=dev.index)
    for i, n in enumerate(lens):
        ctx.fill_random(0, i, 0, n, SEED + i)
    q = torch.randn((B, H, D), device=dev)
    k = torch.randn((B, G, D), device=dev)
    v = torch.randn((B, G, D), device=dev)
    out = torch.zeros((B, H, D), device=dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    times = []
    for i in range(warm + steps):
        ctx.batch_set(list(range(B)), [n + i for n in lens])
        dist.barrier()
        torch.cuda.synchronize()
        ev[0].record(torch.cuda.current_stream(dev))
        ctx.decode_step(0, q, k, v, out=out)
        ev[1].record(torch.cuda.current_stream(dev))
        ev[1].synchronize()
        ms = gather_max(torch, dist, dev, ev[0].elapsed_time(ev[1]))
        if i >= warm:
            times.append(ms)
    ctx.sync()
    ctx.close()
    ms = statistics.median(times)
    nbytes = (sum(lens) + B * (warm + steps // 2)) * BYTES_PER_TOKEN["int8"]      # all 8 heads: the whole job
    gbs = nbytes / ms / 1e6
    return {"metric": METRIC, "value": gbs, "unit": UNIT, "scaling": "strong",
            "workload": "configs[4]: 64 sequences, lengths uniform in [1024, 65536] (seeded), INT8 KV, 1 layer, %d KV head(s) per GPU, no collective" % hc,
            "ms_per_launch": ms, "ms_per_launch_min": min(times), "ms_per_launch_max": max(times), "algorithmic_bytes_per_launch": nbytes,
            "frac_of_aggregate_hbm_peak": gbs / (hbm_peak()[0] * world)}


# ------------------------------------------------------------------------------------- GPU arm: the headline
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from hy3_b200 import Hy3Attn
    from hy3_b200.sharding import make_cuda_sharded_decode

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_layers = args.layers
    ntok0 = args.ntok
    K = args.steps
    ctx = Hy3Attn(kv_dtype=args.kv, n_layers=n_layers, max_batch=1, max_tokens=ntok0 + K + 16 + 256, device=local)
    stream = torch.cuda.Stream(device=dev)
    ctx.set_stream(stream)
    rng = np.random.default_rng(7)
    for l in range(n_layers):
        w = (1.0 + 0.02 * rng.standard_normal((2, 128))).astype(np.float32)
        ctx.set_norm_weights(l, w[0], w[1])
        ctx.fill_random(l, 0, 0, ntok0, SEED + 1000 * rank)
    ctx.sync()
    bytes_per_token = BYTES_PER_TOKEN[args.kv]

    # per-step inputs: the new token's pre-norm q | k | v for every layer, [80][10240] fp32 (reference row layout)
    ROW = H * D + 2 * G * D
    host_in = torch.randn((n_layers, ROW), dtype=torch.float32).pin_memory()
    host_out = torch.empty((n_layers, H * D), dtype=torch.float32).pin_memory()
    with torch.cuda.stream(stream):
        x = host_in.to(dev, non_blocking=True)
        qo = torch.empty((n_layers, 1, H, D), dtype=torch.float32, device=dev)
        out = torch.zeros((n_layers, 1, H, D), dtype=torch.float32, device=dev)
    owner = (rank == world - 1)                      # sequence sharding: the tail rank appends the new token
    sharded = make_cuda_sharded_decode(ctx, 1, n_slots=2) if world > 1 else None
    if world > 1:
        # exchange fused into the kernels: every rank's decode epilogue stores its records into all ranks'
        # gather buffers over NVLink; handles travel once through torch.distributed
        handles = [None] * world
        dist.all_gather_object(handles, ctx.shard_init(rank, world, n_layers, 1))
        ctx.shard_connect(handles)
        dist.barrier()
    side = torch.cuda.Stream(device=dev) if world > 1 else None   # the per-layer exchange runs here, under the next layer's stream of KV

    def layer_views(l):
        row = x[l]
        return (row[:H * D].view(1, H, D), row[H * D:H * D + G * D].view(1, G, D), row[H * D + G * D:].view(1, G, D))

    slot_free = [None, None]

    def enqueue_step(l0=0, l1=None):
        """The launches of layers [l0, l1) of one step on `stream` (captured into a graph once)."""
        for l in range(l0, n_layers if l1 is None else l1):
            q, k, v = layer_views(l)
            if args.two_kernels:
                ctx.append(l, q, k if owner else None, v if owner else None, q_out=qo[l])
                if sharded is None:
                    ctx.decode(l, qo[l], out=out[l])
                else:
                    sharded.step(l, qo[l], out[l])
            elif sharded is None:
                ctx.decode_step(l, q, k, v, out=out[l])        # fused norm+RoPE+quantise/append + attention
            elif not args.nccl_exchange:
                # the exchange is inside the kernel: one launch per layer produces the merged output on every rank
                ctx.decode_step_sharded(l, l, q, k if owner else None, v if owner else None, out=out[l])
            elif args.serial_exchange:
                sharded.step(l, (q, k if owner else None, v if owner else None), out[l])
            else:
                # layers are independent: layer l's all-gather + merge overlap layer l+1's KV stream
                slot = l & 1
                if l >= 2:
                    stream.wait_event(slot_free[slot])          # buffers of layer l-2 have been merged
                sharded.partial(l, (q, k if owner else None, v if owner else None), slot)
                ready = torch.cuda.Event()
                ready.record(stream)
                side.wait_event(ready)
                ctx.set_stream(side)
                with torch.cuda.stream(side):
                    sharded.exchange_merge(slot, out[l])
                    slot_free[slot] = torch.cuda.Event()
                    slot_free[slot].record(side)
                ctx.set_stream(stream)
        if sharded is not None and args.nccl_exchange and not args.serial_exchange and not args.two_kernels:
            for e in slot_free:
                if e is not None:
                    stream.wait_event(e)                         # join the side stream

    def set_positions(step):
        local_slot = ntok0 + step if owner else ntok0 - 1
        global_pos = (ntok0 * world + step) if world > 1 else local_slot
        ctx.batch_set([0], [local_slot], [global_pos])

    stream.synchronize()
    launches_before = ctx.launches
    set_positions(0)
    with torch.cuda.stream(stream):
        enqueue_step()                                # eager warm-up (also warms NCCL)
    stream.synchronize()
    per_step_launches = ctx.launches - launches_before
    graph = torch.cuda.CUDAGraph()
    set_positions(1)
    with torch.cuda.graph(graph, stream=stream):
        enqueue_step()
    stream.synchronize()
    # end-to-end path: ONE graph per step that also holds the host copies.  Inside it the layers run in four quarters on the
    # launching stream while a second, forked stream copies quarter c's inputs host -> device ahead of its launches and its
    # outputs device -> host behind them (a layer needs only its own 41 KB of input and yields 33 KB of output).
    n_chunks = 4 if (n_layers % 4 == 0 and n_layers >= 8 and not (world > 1 and args.nccl_exchange)) else 1
    per_chunk = n_layers // n_chunks
    out2d = out.view(n_layers, H * D)
    copy_stream = torch.cuda.Stream(device=dev)
    graph_e2e = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph_e2e, stream=stream):
        if n_chunks == 1:
            x.copy_(host_in, non_blocking=True)
            enqueue_step()
            host_out.copy_(out2d, non_blocking=True)
        else:
            copy_stream.wait_stream(stream)                       # fork
            h2d, done = [], []
            with torch.cuda.stream(copy_stream):
                for c in range(n_chunks):
                    sl = slice(c * per_chunk, (c + 1) * per_chunk)
                    x[sl].copy_(host_in[sl], non_blocking=True)
                    ev = torch.cuda.Event(); ev.record(copy_stream); h2d.append(ev)
            for c in range(n_chunks):
                stream.wait_event(h2d[c])
                enqueue_step(c * per_chunk, (c + 1) * per_chunk)
                ev = torch.cuda.Event(); ev.record(stream); done.append(ev)
            with torch.cuda.stream(copy_stream):
                for c in range(n_chunks):
                    sl = slice(c * per_chunk, (c + 1) * per_chunk)
                    copy_stream.wait_event(done[c])
                    host_out[sl].copy_(out2d[sl], non_blocking=True)
            stream.wait_stream(copy_stream)                       # join
    stream.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        return gather_max(torch, dist, dev, ms) if world > 1 else ms

    # ---- (1) device-resident throughput: W warm-up steps, then blocks of EXACTLY K timed graph replays, each block
    #          bracketed by barrier + synchronize and timed with CUDA events on the launching stream (max over ranks).
    #          Every block appends at the same K positions (2 .. K+1 past the filled cache), so all blocks do the same work.
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()          # samples clocks / throttle reasons from here to the end of the measurements
    FIRST = 2
    for i in range(args.warmup):
        set_positions(FIRST + i)
        with torch.cuda.stream(stream):
            graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    block_ms = []
    for _ in range(max(1, args.blocks)):
        barrier()
        e0.record(stream)
        for s in range(K):
            set_positions(FIRST + s)
            with torch.cuda.stream(stream):
                graph.replay()
        e1.record(stream)
        barrier()
        block_ms.append(max_over_ranks(e0.elapsed_time(e1)) / K)
    ctx.sync()
    ms_per_step = statistics.median(block_ms)
    tokens_attended = sum(ntok0 + s + 1 for s in range(FIRST, FIRST + K)) / K      # per layer per step
    bytes_per_step = n_layers * tokens_attended * bytes_per_token * world
    value = bytes_per_step / (ms_per_step / 1e3) / 1e9

    # ---- (2) end to end through the public API with HOST buffers (pinned), copies inside the timed region: every step
    #          copies its inputs host -> device, runs, copies its outputs device -> host and synchronises (graph_e2e above).

    def e2e_step(step):
        set_positions(step)
        with torch.cuda.stream(stream):
            graph_e2e.replay()
        stream.synchronize()

    for s in range(2):
        e2e_step(FIRST + s)                           # warm the second path
    barrier()
    t0 = time.perf_counter()
    for s in range(K):
        e2e_step(FIRST + s)
    barrier()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3 / K)
    e2e_value = bytes_per_step / (e2e_ms / 1e3) / 1e9
    e2e_ok = bool(torch.equal(host_out, out2d.cpu())) and bool(torch.isfinite(host_out).all())   # the host buffer holds the step's result

    # ---- (3) the dominant kernel: with the fused step a step IS n_layers launches of it back to back (every layer's
    #          cache is 68 MB and the 80 of them 5.45 GB >> 126 MB L2), so its average launch duration over the timed
    #          region is the block time / launches; with --two-kernels the decode launches are timed alone.
    if per_step_launches == n_layers:
        k_ms = ms_per_step / n_layers
        k_tokens = tokens_attended
        k_how = "median timed block / (%d steps x %d launches)" % (K, n_layers)
    else:
        set_positions(FIRST)
        reps = max(1, 240 // n_layers)
        with torch.cuda.stream(stream):
            def one(l):
                q, k, v = layer_views(l)
                if args.two_kernels:
                    ctx.decode(l, qo[l], out=out[l])
                else:
                    ctx.decode_step(l, q, k if owner else None, v if owner else None, out=out[l])
            for l in range(min(n_layers, 8)):
                one(l)
            e0.record(stream)
            for _ in range(reps):
                for l in range(n_layers):
                    one(l)
            e1.record(stream)
        stream.synchronize()
        k_ms = e0.elapsed_time(e1) / (reps * n_layers)
        k_tokens = ntok0 + FIRST + 1
        k_how = "%d eager launches cycling over the layers" % (reps * n_layers)
    k_bytes = k_tokens * bytes_per_token
    roofline = hbm_roofline(KERNEL_NAME[args.kv], k_bytes / (k_ms / 1e3) / 1e9)
    roofline.update({"us_per_launch": k_ms * 1e3, "algorithmic_bytes_per_launch": k_bytes, "timing": k_how, "traffic": None})
    tr = os.path.join(ROOT, "profiles", "decode_%s_traffic.json" % args.kv)
    if os.path.exists(tr):
        t = json.load(open(tr))
        roofline["traffic"] = t["dram_bytes_per_token_layer"] * k_tokens
        roofline["traffic_source"] = t["source"]
    ctx.sync()

    # ---- (4) N > 1: the in-kernel exchange against the NCCL variant (partials -> all_gather_into_tensor -> merge kernel)
    #          on three layers, same positions; and every rank's merged output against rank 0's, bit for bit
    parity = None
    if world > 1 and not args.two_kernels:
        set_positions(FIRST)
        barrier()
        layers = sorted({0, n_layers // 2, n_layers - 1})
        a = torch.zeros((len(layers), 1, H, D), device=dev)
        b = torch.zeros_like(a)
        with torch.cuda.stream(stream):
            for i, l in enumerate(layers):
                q, k, v = layer_views(l)
                ctx.decode_step_sharded(l, l, q, k if owner else None, v if owner else None, out=a[i])
            for i, l in enumerate(layers):
                q, k, v = layer_views(l)
                sharded.step(l, (q, k if owner else None, v if owner else None), b[i])
        stream.synchronize()
        ctx.sync()
        diff = float((a - b).abs().max().item())
        scale = float(b.abs().max().item())
        everyone = [torch.empty_like(a) for _ in range(world)]
        dist.all_gather(everyone, a)
        same = all(bool(torch.equal(everyone[0], t)) for t in everyone)
        everyone_b = [torch.empty_like(b) for _ in range(world)]
        dist.all_gather(everyone_b, b)
        same_b = all(bool(torch.equal(everyone_b[0], t)) for t in everyone_b)
        diff = gather_max(torch, dist, dev, diff)
        parity = {"layers": layers, "max_abs_vs_nccl_variant": diff, "max_abs_output": scale, "ranks_bit_identical": bool(same),
                  "nccl_variant_ranks_bit_identical": bool(same_b), "finite": bool(torch.isfinite(a).all().item())}

    # ---- (5) secondary workloads
    extra = {}
    if not args.no_prefill:
        if world == 1:
            extra["prefill"] = prefill_section(torch, dev)
            extra["prefill_int8"] = prefill_section(torch, dev, kv="int8")
            extra["prefill_multiturn"] = prefill_section(torch, dev, prompt=1024, prefix=4096)
            extra["decode_fp16"] = decode_cache_type_section(torch, dev, "fp16")
            extra["ragged_batch"] = batch_section(torch, dev, "ragged")
            extra["long_context_int4"] = batch_section(torch, dev, "long")
            extra["long_context_int4_1m"] = batch_section(torch, dev, "long", ntok=1048576)
            extra["reference_gpu_kernel"] = reference_gpu_kernel_section()
        else:
            if world in (2, 4, 8):
                extra["ragged_kv_head_sharded"] = ragged_head_sharded_section(torch, dist, dev, rank, world)
            extra["long_context_int4_sharded"] = {
                "metric": METRIC, "unit": UNIT, "scaling": "strong",
                "workload": "configs[3]: batch 1, INT4 KV, YaRN factor 4, 4 layer caches per step, ONE sequence split by token range over %d GPUs, in-kernel LSE-merge exchange over NVLink peer memory" % world,
                "contexts": [long_sharded_section(torch, dist, dev, rank, world, t) for t in (262144, 1048576)]}
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu:
            cpu = cpu_attention_sample(args.cpu_seconds, False)
            cpu_mt = cpu_attention_sample(min(args.cpu_seconds, 5.0), True)
            cpu["all_threads"] = {k: cpu_mt[k] for k in ("value", "cores", "sample", "ms_per_call")}
        if world == 1:
            how = ""
        elif args.nccl_exchange:
            how = ", sequence-sharded, NCCL all-gather + LSE merge kernel" + (
                " (dependent chain)" if args.serial_exchange else " (exchange of layer l on a side stream under the KV stream of layer l+1)")
        else:
            how = (", sequence-sharded, one launch per layer: the decode kernel's epilogue pushes the rank's records to all ranks "
                   "over NVLink peer memory, waits for theirs and folds (no NCCL call)")
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": args.warmup,
                "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "s8" if args.kv == "int8" else "f16", "data": "synthetic",
                "blocks": {"n": len(block_ms), "steps_each": K, "ms_per_step_median": ms_per_step, "ms_per_step_min": min(block_ms),
                           "ms_per_step_max": max(block_ms)},
                "config": {"workload": WORKLOAD if (world == 1 and args.kv == "int8" and n_layers == N_LAYERS and ntok0 == NTOK)
                           else "%s-KV decode, %d layers x %d positions per GPU, %d GPU(s)%s" % (args.kv, n_layers, ntok0, world, how),
                           "kv_dtype": args.kv, "layers": n_layers, "positions_per_gpu": ntok0, "compute": COMPUTE[args.kv],
                           "l2": "inputs larger than L2: %.2f GB of KV streamed per step, every layer's cache read once" % (bytes_per_step / world / 1e9),
                           "graph": "one CUDA graph of %d launches per step" % per_step_launches},
                "frac_of_hbm_peak": value / world / hbm_peak()[0], "roofline": roofline, "cpu_baseline": cpu,
                "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": host_in.numel() * 4,
                        "d2h_bytes_per_step": host_out.numel() * 4, "host_result_equals_device": e2e_ok,
                        "how": "per step ONE graph: inputs host -> device, %d launches, outputs device -> host, then a synchronise; inside the graph the copies run on a forked stream in %d parts, each ahead of / behind the launches that need / produce it" % (per_step_launches, n_chunks)},
                "gpu_launches": per_step_launches * K, "clocks": clocks}
        if parity is not None:
            line["parity"] = parity
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        # tearing the NCCL communicator down while a captured graph still references it can stall;
        # everything is measured and printed, so leave without the teardown
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)
    del graph
    ctx.close()


def main():
    # the contract is ONE JSON line on stdout: libraries that write to file descriptor 1 themselves (NCCL prints its version
    # there) go to stderr; the JSON line goes to the real stdout
    sys.stdout.flush()
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    sys.stdout = real_stdout
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--blocks", type=int, default=10, help="how many times the block of --steps timed steps is repeated (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kv", default="int8", choices=["int8", "int4", "fp16"])
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--ntok", type=int, default=NTOK)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the secondary workloads (prefill, ragged, long context, sharded variants)")
    ap.add_argument("--prefill-only", action="store_true", help="run only the chunked-prefill measurement and print its JSON object")
    ap.add_argument("--batch-only", choices=["ragged", "long"], help="run only one of the secondary decode workloads and print its JSON object")
    ap.add_argument("--prefill-prompt", type=int, default=8192)
    ap.add_argument("--prefill-prefix", type=int, default=0)
    ap.add_argument("--prefill-kv", default="fp16", choices=["int8", "int4", "fp16"])
    ap.add_argument("--nccl-exchange", action="store_true", help="N>1: exchange the partial records with an NCCL all-gather instead of peer-memory stores from the kernel")
    ap.add_argument("--serial-exchange", action="store_true", help="N>1: all-gather + merge of a layer before the next layer starts (dependent chain)")
    ap.add_argument("--two-kernels", action="store_true", help="append and decode as separate launches instead of the fused step")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.prefill_only:
        import torch
        torch.cuda.set_device(0)
        print(json.dumps(prefill_section(torch, torch.device("cuda", 0), kv=args.prefill_kv, prompt=args.prefill_prompt, prefix=args.prefill_prefix)))
    elif args.batch_only:
        import torch
        torch.cuda.set_device(0)
        print(json.dumps(batch_section(torch, torch.device("cuda", 0), args.batch_only, ntok=args.ntok if args.ntok != NTOK else 262144)))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
