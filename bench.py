#!/usr/bin/env python
"""Benchmark of the Hy3 attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1): decode attention with an INT8 KV cache, batch 1, 80 independent layer caches of
32768 positions each, 64 query heads over 8 KV heads, head_dim 128.  One STEP = one new token:
for each of the 80 layers the fused QK-RMSNorm + RoPE + quantise/append kernel stores the token,
then the split-KV decode kernel attends over all positions (32768 + steps so far).  The 160
launches of a step are replayed as one CUDA graph; lengths live in device memory.
Metric: decode attention KV GB/s = algorithmic KV bytes read per step (ntok x 2080 B per layer,
i.e. codes + fp16 scales of K and V) / time.  Synthetic seeded N(0,1) data, random "weights".

N>1 (weak scaling): every rank holds 32768 positions per layer of ONE sequence of 32768*N tokens
(sequence sharding); per layer ONE launch per rank: the decode kernel's epilogue stores the rank's {m,l,acc}
records into every rank's gather buffer over NVLink peer memory, waits for the others' and folds them
(--nccl-exchange: partial records, NCCL all-gather, merge kernel instead).

Secondary objects in the same JSON line (N=1): "prefill" (configs[2], tensor roofline), "ragged_batch" (configs[4] on one
GPU) and "long_context_int4" (configs[3] on one GPU).

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
SEED = 0x4859335F53454544
METRIC, UNIT = "decode_attn_kv_GBps", "GB/s"
WORKLOAD = ("configs[1]: INT8-KV decode attention, batch 1, 80 independent layer caches x 32768 positions, "
            "64 Q / 8 KV heads, head_dim 128, one token appended per layer per step (fused norm+RoPE+quantise), 1 GPU")


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["hbm_gbs"], "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
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
def cpu_attention_sample(seconds, all_threads):
    """Time the reference CPU attention on a bounded sample of the workload.  Returns a dict with the
    metric value in GB/s of INT8-equivalent KV bytes (tokens x 2080 B), so it is the same unit of work."""
    import numpy as np
    import oracle
    cores = os.cpu_count() or 1
    rng = np.random.default_rng(1)
    if oracle.ref_cpu is not None:
        ntok = 4096           # hy3.c:628-629 caps the reference at 4096 keys; longer inputs are silently truncated
        nl = max(1, min(N_LAYERS, cores // 8 * 2 if all_threads else 1)) if all_threads else 1
        K = rng.standard_normal((ntok, G, D)).astype(np.float32)
        V = rng.standard_normal((ntok, G, D)).astype(np.float32)
        for l in range(nl):
            oracle.ref_cpu.load_layer(K, V, l)
        q = rng.standard_normal((nl, H, D)).astype(np.float32)
        if all_threads:
            fn = lambda: oracle.ref_cpu.attention_layers(q, ntok)
            threads = min(cores, nl * 8, oracle.ref_cpu.max_threads())
        else:
            fn = lambda: oracle.ref_cpu.attention(q[0], ntok, 0)
            threads = 1
        kind = "reference"
        sample = ("hy3.c attention() as shipped (-O3 -ffast-math), fp32 KV, %d layer(s) x first %d of 32768 positions "
                  "(the reference caps at 4096 keys), %d thread(s)" % (nl, ntok, threads))
    else:
        ntok, nl, threads, kind = NTOK, 1, 1, "port"
        K = rng.standard_normal((ntok, G, D)).astype(np.float32)
        V = rng.standard_normal((ntok, G, D)).astype(np.float32)
        q = rng.standard_normal((1, H, D)).astype(np.float32)
        fn = lambda: oracle.attention(q[0], K, V)
        sample = "C restatement of hy3.c attention(), fp32 KV, 1 layer x 32768 positions, 1 thread"
    fn()
    times = []
    t_end = time.perf_counter() + seconds
    while time.perf_counter() < t_end or len(times) < 3:
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    best = statistics.median(times)
    gbs = nl * ntok * INT8_BYTES_PER_TOKEN_LAYER / best / 1e9
    return {"value": gbs, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample,
            "ms_per_call": best * 1e3, "host_cores": cores, "fp32_kv_GBps": nl * ntok * 2 * G * D * 4 / best / 1e9,
            "layers": nl, "ntok": ntok}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step = None
    base = cpu_attention_sample(0.0, True)        # warm + shape
    import oracle  # noqa: F401
    # one "step" = one pass of the bounded sample; W warm-up, K timed
    import numpy as np  # noqa: F401
    times = []
    for i in range(args.warmup + args.steps):
        r = cpu_attention_sample(0.0, True)
        if i >= args.warmup:
            times.append(r["ms_per_call"])
    per_step = sum(times) / len(times)
    value = base["layers"] * base["ntok"] * INT8_BYTES_PER_TOKEN_LAYER / (per_step / 1e3) / 1e9
    cb = {k: base[k] for k in ("unit", "cores", "kind", "sample")}
    cb["value"] = value
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": per_step, "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD},
                      "cpu_baseline": cb, "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "gpu_launches": 0}))


# ------------------------------------------------------------------------------------- GPU arm
def batch_section(torch, dev, kind):
    """Secondary decode workloads, one layer each, device-timed back-to-back fused steps:
    'ragged'  -- configs[4] on one GPU: 64 sequences, lengths 1024 + (rng % 64513) (seeded), INT8 KV, one token per
                 sequence per step (all 8 KV heads on this GPU);
    'long'    -- configs[3] on one GPU: batch 1, INT4 KV, 262 144 positions, YaRN factor 4 (attn_factor on q and k)."""
    import numpy as np
    from hy3_b200 import Hy3Attn
    rng = np.random.default_rng(SEED)
    if kind == "ragged":
        kv, lens = "int8", [int(1024 + rng.integers(0, 64513)) for _ in range(64)]
        what = "configs[4]: 64 sequences, lengths uniform in [1024, 65536] (seeded), INT8 KV, 1 layer, all 8 KV heads on one GPU"
    else:
        kv, lens = "int4", [262144]
        what = "configs[3]: batch 1, INT4 KV, 262144 positions, YaRN factor 4, 1 layer, unsharded"
    B = len(lens)
    steps = 24
    ctx = Hy3Attn(kv_dtype=kv, n_layers=1, max_seqs=B, max_batch=B, max_tokens=sum(lens) + (steps + 129) * B, max_tokens_per_seq=max(lens) + steps + 129, device=dev.index)
    if kind == "long":
        inv = (1.0 / (11158840.0 ** (np.arange(64) / 64.0))).astype(np.float32)
        ctx.set_rope(inv / 4.0, 1.0 + 0.1 * np.log(4.0))      # every frequency interpolated: the speed does not depend on the blend
    for i, n in enumerate(lens):
        ctx.fill_random(0, i, 0, n, SEED + i)
    q = torch.randn((B, H, D), device=dev)
    k = torch.randn((B, G, D), device=dev)
    v = torch.randn((B, G, D), device=dev)
    out = torch.zeros((B, H, D), device=dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    t = 0
    for _ in range(4):                                          # warm-up
        ctx.batch_set(list(range(B)), [n + t for n in lens]); ctx.decode_step(0, q, k, v, out=out); t += 1
    torch.cuda.synchronize()
    times = []
    for _ in range(steps - 4):
        ctx.batch_set(list(range(B)), [n + t for n in lens])
        ev[0].record(torch.cuda.current_stream(dev))
        ctx.decode_step(0, q, k, v, out=out)
        ev[1].record(torch.cuda.current_stream(dev))
        ev[1].synchronize()
        times.append(ev[0].elapsed_time(ev[1]))
        t += 1
    ctx.sync()
    ctx.close()
    ms = statistics.median(times)
    per_tok = {"int8": 2080, "int4": 1056, "fp16": 4096}[kv]
    nbytes = (sum(lens) + B * (4 + (steps - 4) // 2)) * per_tok
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = json.load(open(p))["hbm_gbs"] if os.path.exists(p) else 6650.0
    gbs = nbytes / ms / 1e6
    return {"metric": METRIC, "value": gbs, "unit": UNIT, "workload": what, "ms_per_launch": ms, "algorithmic_bytes_per_launch": nbytes,
            "l2": "%.2f GB streamed per launch, far beyond L2" % (nbytes / 1e9),
            "roofline": {"bound": "hbm", "kernel": "hy3a_decode_kernel<%s>" % kv, "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                         "frac_of_nominal_8TBs": gbs / 8000.0,
                         "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if os.path.exists(p) else "fallback 6.65 TB/s"}}


def prefill_section(torch, dev, kv="fp16", prompt=8192, chunk=512):
    """Secondary metric: chunked causal prefill attention, an 8192-token prompt in 512-token chunks,
    FP16 KV cache, 64 Q / 8 KV heads, one layer (configs[2]).  TFLOP/s = 4*128*64*sum(pos+1) / device time
    of the attention calls (conversion of pages not yet in the fp16 operand mirror, if any, + tcgen05 kernel); the fused
    append -- which also writes the chunk's rows through into the mirror -- is timed separately and reported beside it."""
    from hy3_b200 import Hy3Attn
    ctx = Hy3Attn(kv_dtype=kv, n_layers=1, max_batch=chunk, max_tokens=prompt + 256, device=dev.index)
    q = torch.randn((prompt, H, D), device=dev)
    k = torch.randn((prompt, G, D), device=dev)
    v = torch.randn((prompt, G, D), device=dev)
    q16 = torch.empty((chunk, H, D), dtype=torch.float16, device=dev)
    out = torch.zeros((chunk, H, D), device=dev)

    def run():
        att, app = [], []
        for c in range(prompt // chunk):
            b = c * chunk
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ctx.batch_set([0] * chunk, list(range(b, b + chunk)))
            ev[0].record()
            ctx.append(0, q[b:b + chunk], k[b:b + chunk], v[b:b + chunk], q_out=False, q_out16=q16)
            ev[1].record()
            ctx.prefill(0, 0, b, q16, out=out)
            ev[2].record()
            att.append((ev[1], ev[2])); app.append((ev[0], ev[1]))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in att), sum(a.elapsed_time(b) for a, b in app)
    for _ in range(3):
        run()
    att_ms, app_ms = min(run() for _ in range(3))
    ctx.sync()
    launches = ctx.launches
    ctx.close()
    pairs = sum(c * chunk + i + 1 for c in range(prompt // chunk) for i in range(chunk))
    flops = 4.0 * D * H * pairs
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = json.load(open(p))["bf16_tflops"] if os.path.exists(p) else 1590.0
    tf = flops / att_ms / 1e9
    return {"metric": "prefill_attn_TFLOPs", "value": tf, "unit": "TFLOP/s", "workload": "configs[2]: %d-token prompt in %d-token chunks, %s KV, 1 layer" % (prompt, chunk, kv),
            "attention_ms_per_layer": att_ms, "append_ms_per_layer": app_ms, "algorithmic_tflop_per_layer": flops / 1e12,
            "roofline": {"bound": "tensor", "kernel": "hy3a_prefill_kernel", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                         "frac_of_nominal_2250": tf / 2250.0,
                         "peak_source": "measured (MEASURED_PEAKS.json bf16_tflops, burst)" if os.path.exists(p) else "fallback 1.59 PFLOP/s"},
            "gpu_launches_total": launches}


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
    total_steps = args.warmup + args.steps + 8
    n_layers = args.layers
    ntok0 = args.ntok
    ctx = Hy3Attn(kv_dtype=args.kv, n_layers=n_layers, max_batch=1, max_tokens=ntok0 + total_steps + 256, device=local)
    stream = torch.cuda.Stream(device=dev)
    ctx.set_stream(stream)
    rng = np.random.default_rng(7)
    for l in range(n_layers):
        w = (1.0 + 0.02 * rng.standard_normal((2, 128))).astype(np.float32)
        ctx.set_norm_weights(l, w[0], w[1])
        ctx.fill_random(l, 0, 0, ntok0, SEED + 1000 * rank)
    ctx.sync()
    bytes_per_token = {"int8": 2080, "int4": 1056, "fp16": 4096}[args.kv]

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
    if world > 1 and not args.nccl_exchange:
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

    def enqueue_step():
        """All launches of one step on `stream` (captured into a graph once)."""
        for l in range(n_layers):
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
        if sharded is not None and not args.serial_exchange and not args.two_kernels:
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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- (1) device-resident throughput: W warm-up + K timed graph replays
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()          # samples clocks / throttle reasons from here to the end of the measurements
    step_no = 2
    for _ in range(args.warmup):
        set_positions(step_no); step_no += 1
        with torch.cuda.stream(stream):
            graph.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first_step = step_no
    e0.record(stream)
    for _ in range(args.steps):
        set_positions(step_no); step_no += 1
        with torch.cuda.stream(stream):
            graph.replay()
    e1.record(stream)
    barrier()
    ms_total = e0.elapsed_time(e1)
    ctx.sync()
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    tokens_attended = sum(ntok0 + s + 1 for s in range(first_step, first_step + args.steps)) / args.steps  # per layer per step
    bytes_per_step = n_layers * tokens_attended * bytes_per_token * world
    value = bytes_per_step / (ms_per_step / 1e3) / 1e9

    # ---- (2) end to end through the public API with HOST buffers (pinned), copies inside the timed region
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        set_positions(step_no); step_no += 1
        with torch.cuda.stream(stream):
            x.copy_(host_in, non_blocking=True)
            graph.replay()
            host_out.copy_(out.view(n_layers, H * D), non_blocking=True)
        stream.synchronize()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = bytes_per_step / (e2e_ms / 1e3) / 1e9

    # ---- (3) the dominant kernel alone: decode launches cycling over the layers (each layer's cache is
    #          68 MB and the 80 of them 5.45 GB >> 126 MB L2), CUDA events on the launching stream
    set_positions(step_no)
    reps = max(1, 240 // n_layers)
    with torch.cuda.stream(stream):
        def one(l):
            q, k, v = layer_views(l)
            if args.two_kernels:
                ctx.decode(l, qo[l], out=out[l])
            else:
                ctx.decode_step(l, q, k if owner else None, v if owner else None, out=out[l])   # the kernel a step launches
        for l in range(min(n_layers, 8)):
            one(l)
        e0.record(stream)
        for _ in range(reps):
            for l in range(n_layers):
                one(l)
        e1.record(stream)
    stream.synchronize()
    k_ms = e0.elapsed_time(e1) / (reps * n_layers)
    k_bytes = (ntok0 + step_no + 1) * bytes_per_token
    peak, peak_src = peaks()
    achieved = k_bytes / (k_ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "kernel": "hy3a_decode_kernel<%s>" % args.kv, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "frac_of_nominal_8TBs": achieved / 8000.0, "peak_source": peak_src,
                "us_per_launch": k_ms * 1e3, "algorithmic_bytes_per_launch": k_bytes, "traffic": None}
    tr = os.path.join(ROOT, "profiles", "decode_%s_traffic.json" % args.kv)
    if os.path.exists(tr):
        t = json.load(open(tr))
        roofline["traffic"] = t["dram_bytes_per_token_layer"] * (ntok0 + step_no + 1)
        roofline["traffic_source"] = t["source"]
    ctx.sync()
    prefill = prefill_section(torch, dev) if (rank == 0 and world == 1 and not args.no_prefill) else None
    extra = {}
    if rank == 0 and world == 1 and not args.no_prefill:
        for kind in ("ragged", "long"):
            extra[kind] = batch_section(torch, dev, kind)
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu:
            cpu = cpu_attention_sample(args.cpu_seconds, False)
            cpu_mt = cpu_attention_sample(min(args.cpu_seconds, 5.0), True)
            cpu["all_threads"] = {k: cpu_mt[k] for k in ("value", "cores", "sample", "ms_per_call")}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f16", "data": "synthetic",
                "config": {"workload": WORKLOAD if (world == 1 and args.kv == "int8" and n_layers == N_LAYERS and ntok0 == NTOK)
                           else "%s-KV decode, %d layers x %d positions per GPU, %d GPU(s)%s" % (
                               args.kv, n_layers, ntok0, world, (", sequence-sharded, " + (("NCCL all-gather + LSE merge kernel" + (" (exchange of layer l on a side stream under the KV stream of layer l+1)" if not args.serial_exchange else " (dependent chain)")) if args.nccl_exchange else "one launch per layer: the decode kernel's epilogue pushes the rank's records to all ranks over NVLink peer memory, waits for theirs and folds (no NCCL call)")) if world > 1 else ""),
                           "kv_dtype": args.kv, "layers": n_layers, "positions_per_gpu": ntok0, "compute": "fp16 mma.sync, fp32 accumulate/softmax",
                           "l2": "inputs larger than L2: %.2f GB of KV streamed per step, every layer's cache read once" % (bytes_per_step / world / 1e9),
                           "graph": "one CUDA graph of %d launches per step" % per_step_launches},
                "frac_of_hbm_peak": value / world / peak, "roofline": roofline, "cpu_baseline": cpu,
                "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": host_in.numel() * 4,
                        "d2h_bytes_per_step": host_out.numel() * 4},
                "gpu_launches": per_step_launches * args.steps, "clocks": clocks, "prefill": prefill,
                "ragged_batch": extra.get("ragged"), "long_context_int4": extra.get("long")}
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
    if os.environ.get("HY3_BENCH_WATCHDOG"):     # development aid: dump the Python stacks if the run stalls
        import faulthandler
        faulthandler.dump_traceback_later(int(os.environ["HY3_BENCH_WATCHDOG"]), exit=True)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kv", default="int8", choices=["int8", "int4", "fp16"])
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--ntok", type=int, default=NTOK)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the secondary chunked-prefill measurement")
    ap.add_argument("--prefill-only", action="store_true", help="run only the chunked-prefill measurement and print its JSON object")
    ap.add_argument("--batch-only", choices=["ragged", "long"], help="run only one of the secondary decode workloads and print its JSON object")
    ap.add_argument("--prefill-prompt", type=int, default=8192)
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
        print(json.dumps(prefill_section(torch, torch.device("cuda", 0), kv=args.prefill_kv, prompt=args.prefill_prompt)))
    elif args.batch_only:
        import torch
        torch.cuda.set_device(0)
        print(json.dumps(batch_section(torch, torch.device("cuda", 0), args.batch_only)))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
