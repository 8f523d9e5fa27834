"""Benchmark of the algebraic forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (benchmark configuration 5 at the length its target is quoted on): asinh-power
attention forward, bf16, causal, batch 1 x 16 heads x head_dim 128 x seq 8192 PER GPU,
range-guarded, sink present, n=16, c=8.  Units are (batch, head) pairs; at N GPUs every
rank runs its own 16 units (weak scaling, no collective on the attention path).
metric = causal forward TFLOP/s with the reference's FLOP convention 4*B*H*T^2*D/2.

One JSON line on stdout (rank 0).  Besides the contract keys it carries
  roofline       : the attention kernel alone, timed with CUDA events, against the measured
                   dense bf16 peak of MEASURED_PEAKS.json
  roofline_head  : the fused Alg-CE head of configuration 2 the same way (N = 1 only)
  cpu_baseline   : the CPU oracle timed on this host on a bounded sample of the headline workload
                   (configurations 1 and 2 in full under extra.cpu_configs)
  e2e            : the same metric through the public Python call with pinned HOST buffers,
                   host->device copies of q,k,v and the device->host copy of o inside the
                   timed region
  extra          : the other hot-path kernels and the prefill models with their own fractions; at
                   N > 1 the vocabulary-sharded head, the batch-split prefill, the heads-partitioned
                   attention of configuration 5, and `parity_multi_gpu` (what was exchanged,
                   compared with a single-rank recomputation on rank 0).
`--impl reference` times the reference's CPU path (its restatement in oracle/, or the reference's
own JAX functions if `import jax` works on the box) on a bounded sample per step, rank 0 only.
"""

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

ATTN = dict(B=1, H=16, T=8192, D=128, n=16, c=8.0)
HEAD = dict(N=8192, d=768, V=50304, n=8, c=2.0, target_hi=50257)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the attention kernel at the headline
# shape, from the ncu capture summarised in profiles/attn_tc_kernel_config5_seq8192.md (the guarded
# call's launch: 165.1 MB read, of which the in-kernel guard statistics add what L2 does not hold,
# 14.7 MB written).
ATTN_DRAM_TRAFFIC_BYTES = 179.9e6
REPS = 5                      # repetitions of the timed region; the median is reported


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


def attn_flops(B, H, T, D):
    return 4.0 * B * H * T * T * D / 2.0


def make_attn_inputs(seed, shape):
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn(shape, generator=g).bfloat16() for _ in range(3))


def reference_attention_fn():
    """(callable, kind): the reference's own dense attention under JAX on CPU when JAX can be
    imported on this box (also from a baseline/_ref install), else its CPU restatement."""
    try:
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if os.path.isdir(ref_dir) and ref_dir not in sys.path:
            sys.path.insert(0, ref_dir)
        os.environ.setdefault("JAX_PLATFORMS", "cpu")
        import jax.numpy as jnp                                   # noqa: F401
        from algebraic import algebraic as REF

        def run(q, k, v, sink):
            out = REF.asinh_attention(jnp.asarray(q.float().numpy()), jnp.asarray(k.float().numpy()),
                                      jnp.asarray(v.float().numpy()), n=ATTN["n"], c=ATTN["c"],
                                      sink_logit=jnp.asarray(sink.numpy()).reshape(1, -1, 1, 1))
            out.block_until_ready()
        return run, "reference"
    except Exception:
        from oracle import algebraic_ref as R

        def run(q, k, v, sink):
            R.asinh_attention(q, k, v, n=ATTN["n"], c=ATTN["c"], sink_logit=sink, row_block=1024)
        return run, "port"


def run_reference_arm(args, rank):
    """The reference's CPU implementation of the path.  Each step is a bounded sample: one
    (batch, head) unit at full T."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    fn, kind = reference_attention_fn()
    T, D = ATTN["T"], ATTN["D"]
    q, k, v = make_attn_inputs(0, (1, 1, T, D))
    sink = torch.zeros(1)
    for _ in range(max(1, min(args.warmup, 2))):
        fn(q, k, v, sink)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn(q, k, v, sink)
    dt = (time.perf_counter() - t0) / args.steps
    val = attn_flops(1, 1, T, D) / dt / 1e12
    sample = f"1 of {ATTN['B'] * ATTN['H']} (batch, head) units per step at full T={T}, D={D}"
    out = {"impl": "reference", "metric": "asinh_attn_fwd_tflops", "value": val, "unit": "TFLOP/s",
           "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
           "data": "synthetic", "config": workload_config(args.gpus),
           "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
           "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "note": "reference asinh_attention under JAX on CPU" if kind == "reference"
                   else "CPU restatement of src/algebraic/algebraic.py asinh_attention (JAX not importable here)"}
    print(json.dumps(out), flush=True)


def workload_config(n_gpus):
    return {"workload": "config 5 @ seq 8192: asinh attention fwd, bf16, causal, guarded, sink",
            "batch_per_gpu": ATTN["B"], "heads": ATTN["H"], "seq_len": ATTN["T"], "head_dim": ATTN["D"],
            "n": ATTN["n"], "c": ATTN["c"], "units_per_gpu": ATTN["B"] * ATTN["H"],
            "parallelism": f"(batch,head) units x{n_gpus}, no collective",
            "l2_policy": "two input sets alternate (2 x 134 MB > 126 MB L2)",
            "flop_convention": "4*B*H*T^2*D/2", "timing": f"median of {REPS} regions of --steps steps"}


def cuda_time(fn, iters, sync):
    """Average milliseconds per call of fn over `iters` back-to-back calls, CUDA events on the
    current stream, synchronised on both sides."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    start.record()
    for i in range(iters):
        fn(i)
    end.record()
    sync()
    return start.elapsed_time(end) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel", default="auto", choices=["auto", "mma", "tcgen05"],
                    help="attention/head kernel family (auto = tcgen05 where it applies)")
    ap.add_argument("--skip-extra", action="store_true", help="headline workload only")
    ap.add_argument("--prefill-only", default=None, choices=["125m", "350m", "1b"],
                    help="profiling aid: run only this prefill model in the extra section")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch.distributed as dist
    import algebraic_transformer_b200 as A
    from algebraic_transformer_b200 import _lib
    from algebraic_transformer_b200.dist import init_from_env, vocab_shard

    rank, world, local = init_from_env("nccl")
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}; using {world}", file=sys.stderr)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    lib = _lib.load()
    pk = peaks()

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def median_time(fn, iters):
        """Median over REPS timed regions of `iters` steps each (max over ranks per region)."""
        return statistics.median(max_over_ranks(cuda_time(fn, iters, sync)) for _ in range(REPS))

    # ---------------- headline: guarded attention, inputs resident in HBM ----------------
    B, H, T, D = ATTN["B"], ATTN["H"], ATTN["T"], ATTN["D"]
    host_sets = [make_attn_inputs(1000 * rank + s, (B, H, T, D)) for s in range(2)]
    dev_sets = [tuple(t.to(dev) for t in hs) for hs in host_sets]
    outs = [torch.empty((B, H, T, D), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    sink = torch.zeros(H, dtype=torch.float32, device=dev)

    def attn_step(i):
        q, k, v = dev_sets[i & 1]
        A.flash_attention(q, k, v, sink, kind="asinh", n=ATTN["n"], c=ATTN["c"], range_guard=True,
                          shift=False, impl=args.kernel, out=outs[i & 1])

    from algebraic_transformer_b200.clocks import NvmlSampler
    sampler = NvmlSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(args.warmup):
        attn_step(i)
    # keep the GPU under the same load for a moment before timing, so that the clocks the
    # timed steps see are the steady ones (untimed, on top of the W warm-up steps)
    t_hold = time.perf_counter()
    while time.perf_counter() - t_hold < 0.25:
        for i in range(8):
            attn_step(i)
        torch.cuda.synchronize()
    launches0 = lib.alg_kernel_launches()
    t_region0 = time.perf_counter()
    ms = median_time(attn_step, args.steps)
    t_region1 = time.perf_counter()
    launches = (lib.alg_kernel_launches() - launches0) // REPS
    flops_rank = attn_flops(B, H, T, D)
    value = flops_rank * world / (ms * 1e-3) / 1e12

    # the attention kernel alone (no guard statistics, no stand-by launch of the stable kernel)
    def attn_only(i):
        q, k, v = dev_sets[i & 1]
        A.ops._attention_unshifted_unclamped(q, k, v, sink, n=ATTN["n"], c=ATTN["c"], impl=args.kernel,
                                             out=outs[i & 1])

    for i in range(3):
        attn_only(i)
    t_k0 = time.perf_counter()
    ms_kernel = median_time(attn_only, args.steps)
    t_k1 = time.perf_counter()
    clocks, clocks_kernel = None, None
    if rank == 0:
        sampler.stop()
        clocks = sampler.summary(t_region0, t_region1)
        clocks_kernel = sampler.summary(t_k0, t_k1)
    peak_tf = float(pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    achieved = flops_rank / (ms_kernel * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                "frac": achieved / peak_tf, "traffic": ATTN_DRAM_TRAFFIC_BYTES,
                "kernel_ms": ms_kernel, "peak_source": pk["_source"] + " (burst bf16 GEMM)",
                "algorithmic_flops_per_launch": flops_rank,
                "sm_mhz": clocks_kernel["sm_mhz"] if clocks_kernel else None,
                "kernel_ms_x_sm_mhz": ms_kernel * clocks_kernel["sm_mhz"] if clocks_kernel and clocks_kernel["sm_mhz"] else None}

    # ---------------- e2e: host buffers, copies inside the timed region --------------------
    pinned = [tuple(t.pin_memory() for t in hs) for hs in host_sets]
    o_host = torch.empty((B, H, T, D), dtype=torch.bfloat16).pin_memory()
    # Every step copies its own q, k, v from pinned host memory, runs the public call on them
    # and copies its output back.  Steps are software-pipelined over three streams (upload of
    # step i+1 and download of step i-1 overlap the kernels of step i) with two sets of device
    # staging buffers; the timed region ends when the last download has landed.
    stage = [[torch.empty((B, H, T, D), dtype=torch.bfloat16, device=dev) for _ in range(3)] for _ in range(2)]
    o_dev = [torch.empty((B, H, T, D), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    s_up, s_down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    ev_up = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_down = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        b2 = i & 1
        cur = torch.cuda.current_stream()
        s_up.wait_event(ev_done[b2])                       # staging set b2 is free once step i-2 computed
        with torch.cuda.stream(s_up):
            for dst, src in zip(stage[b2], pinned[b2]):
                dst.copy_(src, non_blocking=True)
            ev_up[b2].record()
        cur.wait_event(ev_up[b2])
        cur.wait_event(ev_down[b2])                        # o_dev[b2] has been downloaded (step i-2)
        A.flash_attention(stage[b2][0], stage[b2][1], stage[b2][2], sink, kind="asinh", n=ATTN["n"], c=ATTN["c"],
                          range_guard=True, impl=args.kernel, out=o_dev[b2])
        ev_done[b2].record()
        s_down.wait_event(ev_done[b2])
        with torch.cuda.stream(s_down):
            o_host.copy_(o_dev[b2], non_blocking=True)
            ev_down[b2].record()

    def e2e_loop(n):
        for i in range(n):
            e2e_step(i)
        torch.cuda.current_stream().wait_stream(s_down)    # the last result is on the host

    e2e_loop(3)
    e2e_steps = max(3, min(args.steps, 40))              # fill and drain of the three-stream pipeline are inside the region
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    ev0.record()
    e2e_loop(e2e_steps)
    ev1.record()
    sync()
    ms_e2e = max_over_ranks(ev0.elapsed_time(ev1) / e2e_steps)
    tensor_bytes = B * H * T * D * 2
    e2e = {"value": flops_rank * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": 3 * tensor_bytes, "d2h_bytes_per_step": tensor_bytes, "ms_per_step": ms_e2e}
    del stage, o_dev, pinned, o_host, host_sets, dev_sets, outs
    torch.cuda.empty_cache()

    extra, roofline_head = {}, None
    if not args.skip_extra:
        extra, roofline_head = run_extra(A, dist, vocab_shard, dev, rank, world, sync, max_over_ranks, pk, args)

    cpu_baseline = None
    if rank == 0 and world == 1:
        cpu_baseline = time_cpu_baseline()
        if not args.skip_extra:
            extra["cpu_configs"] = time_cpu_configs()

    if rank == 0:
        out = {"metric": "asinh_attn_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
               "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
               "config": workload_config(world), "roofline": roofline, "roofline_head": roofline_head,
               "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
               "frac_of_bf16_peak_whole_step": value / world / peak_tf, "extra": extra,
               "library": os.path.relpath(_lib.LIB_PATH, ROOT), "kernel_family": args.kernel}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def time_cpu_baseline():
    """The CPU path on a bounded sample of the headline workload: a few (batch, head) units
    at full sequence length, all host threads."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    fn, kind = reference_attention_fn()
    T, D = ATTN["T"], ATTN["D"]
    q, k, v = make_attn_inputs(0, (1, 1, T, D))
    sink = torch.zeros(1)
    fn(q[:, :, :1024], k[:, :, :1024], v[:, :, :1024], sink)          # warm the threads
    units, t0 = 0, time.perf_counter()
    while units < 4 and (time.perf_counter() - t0 < 20.0 or units == 0):
        fn(q, k, v, sink)
        units += 1
    dt = time.perf_counter() - t0
    return {"value": attn_flops(1, units, T, D) / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"{units} of {ATTN['B'] * ATTN['H']} (batch, head) units at full T={T}, D={D} ({dt:.1f} s of CPU work)"}


def time_cpu_configs():
    """Benchmark configurations 1 and 2 in full on the host cores (the CPU oracle): configuration 1 is
    the reference's own CPU-runnable case; configuration 2 forms the dense 8192 x 50304 fp32 logits."""
    from oracle import algebraic_ref as R
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    out = {"cores": cores, "kind": "port"}
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn((4, 12, 1024, 64), generator=g) for _ in range(3))
    cos, sin = R.cayley_table_geometric(64, 1024)
    gs = torch.Generator().manual_seed(1)
    sink = torch.randn(12, generator=gs) * 0.02
    ones = torch.ones(64)

    def config1():
        qn = R.apply_rotary(R.rms_norm(q, ones, 1e-5), cos, sin)
        kn = R.apply_rotary(R.rms_norm(k, ones, 1e-5), cos, sin)
        return R.asinh_attention(qn, kn, v, n=16, c=8.0, sink_logit=sink)

    config1()
    ts = []
    for _ in range(3):
        t0 = time.perf_counter()
        config1()
        ts.append(time.perf_counter() - t0)
    s1 = statistics.median(ts)
    out["config1_attention_layer_fp32"] = {"s": s1, "tflops": attn_flops(4, 12, 1024, 64) / s1 / 1e12}
    N, d, V = HEAD["N"], HEAD["d"], HEAD["V"]
    h = torch.randn((N, d), generator=g).bfloat16()
    E = torch.randn((V, d), generator=g) * 0.02
    t = torch.randint(0, HEAD["target_hi"], (N,), generator=g)
    t0 = time.perf_counter()
    R.head_loss_dense(h, E, t, HEAD["n"], HEAD["c"])
    s2 = time.perf_counter() - t0
    out["config2_dense_head"] = {"s": s2, "tflops": 2.0 * N * d * V / s2 / 1e12}
    return out


def run_extra(A, dist, vocab_shard, dev, rank, world, sync, max_over_ranks, pk, args):
    """Head (vocab-sharded, with its all-reduce at N>1), prefill models, heads-partitioned attention,
    and at N=1 the longer sequences, qk_rms, decode, projections and backward kernels."""
    from algebraic_transformer_b200.dist import unit_shard
    extra, parity = {}, {}
    peak_tf = float(pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    peak_bw = float(pk.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    iters = max(5, min(args.steps, 20))

    def rel(a, b):
        a, b = a.double(), b.double()
        return float((a - b).norm() / b.norm().clamp_min(1e-300))

    # ---- fused Alg-CE head: benchmark configuration 2, vocabulary sharded over ranks ----
    N, d, V = HEAD["N"], HEAD["d"], HEAD["V"]
    g = torch.Generator().manual_seed(0)
    h = torch.randn((N, d), generator=g).bfloat16().to(dev)
    lo, cnt = vocab_shard(V, rank, world)
    shards = []                                             # every rank can rebuild every shard (seeded)
    for r in range(world):
        ge = torch.Generator().manual_seed(1 + r)
        shards.append((torch.randn((vocab_shard(V, r, world)[1], d), generator=ge) * 0.02).bfloat16())
    e = shards[rank].to(dev)
    t = torch.randint(0, HEAD["target_hi"], (N,), generator=g).to(torch.int32).to(dev)
    stats = torch.empty((2, N), dtype=torch.float32, device=dev)

    def head_step(i):
        A.head_statistic(h, e, t, n=HEAD["n"], c=HEAD["c"], vocab_offset=lo, vocab_total=V, impl=args.kernel,
                         out=stats)
        if world > 1:
            dist.all_reduce(stats, op=dist.ReduceOp.SUM)
        return A.head_finalize(stats, n=HEAD["n"], c=HEAD["c"], vocab_total=V)

    def head_kernel_only(i):
        A.head_statistic(h, e, t, n=HEAD["n"], c=HEAD["c"], vocab_offset=lo, vocab_total=V, impl=args.kernel,
                         out=stats)

    for i in range(3):
        head_step(i)
    ms_head = max_over_ranks(cuda_time(head_step, iters, sync))
    ms_head_k = max_over_ranks(cuda_time(head_kernel_only, iters, sync))
    fl = 2.0 * N * d * V
    fl_local = 2.0 * N * d * cnt
    extra["alg_ce_head"] = {
        "workload": f"config 2, vocab sharded x{world}", "tflops": fl / (ms_head * 1e-3) / 1e12, "ms_per_step": ms_head,
        "kernel_ms": ms_head_k, "kernel_tflops_per_gpu": fl_local / (ms_head_k * 1e-3) / 1e12,
        "frac_of_bf16_peak": fl_local / (ms_head_k * 1e-3) / 1e12 / peak_tf,
        "collective": "none" if world == 1 else "NCCL all-reduce of (2,N) fp32", "logits_bytes_written": 0}
    roofline_head = None
    if world == 1:
        roofline_head = {"bound": "tensor", "achieved": fl / (ms_head_k * 1e-3) / 1e12, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": fl / (ms_head_k * 1e-3) / 1e12 / peak_tf, "kernel_ms": ms_head_k,
                         "call_ms": ms_head, "traffic": 94.9e6, "logits_bytes_written": 0,
                         "workload": "config 2: N=8192 d=768 V=50304 bf16"}
    if world > 1:
        # what the exchange produced against a single-rank recomputation over the whole vocabulary
        pt_nccl = head_step(0)[1].clone()
        e_full = torch.cat(shards).to(dev)
        single = A.head_statistic(h, e_full, t, n=HEAD["n"], c=HEAD["c"], vocab_total=V, impl=args.kernel)
        pt_single = A.head_finalize(single, n=HEAD["n"], c=HEAD["c"], vocab_total=V)[1]
        parity["head_nccl_pt_rel_l2"] = rel(pt_nccl, pt_single)
        try:
            from algebraic_transformer_b200.dist import HeadExchange
            ex = HeadExchange(dist.group.WORLD, N, dev)

            def head_fused_step(i):
                return A.ops._fused_head_exchange(h, e, t, ex, n=HEAD["n"], c=HEAD["c"], vocab_offset=lo, vocab_total=V,
                                                  want_nll=False, impl=args.kernel)

            for i in range(3):
                head_fused_step(i)
            ms_fx = max_over_ranks(cuda_time(head_fused_step, iters, sync))
            pt_fx = head_fused_step(0)[1]
            torch.cuda.synchronize()
            parity["head_exchange_pt_rel_l2"] = rel(pt_fx, pt_single)
            extra["alg_ce_head_fused_exchange"] = {
                "tflops": fl / (ms_fx * 1e-3) / 1e12, "ms_per_step": ms_fx,
                "collective": "none: one kernel does split reduction, NVLink peer stores, flag wait, telemetry"}
            del ex
        except Exception as err:                         # symmetric memory unavailable on this box
            extra["alg_ce_head_fused_exchange"] = {"unavailable": repr(err)[:200]}
        del e_full, single
    del h, e, t, stats, shards

    # ---- configuration 5 with the heads partitioned over the ranks (strong scaling of one 16-head problem) ----
    part = {}
    for T in (8192, 32768):
        u0, un = unit_shard(ATTN["H"], rank, world)
        q, k, v = (x.to(dev) for x in make_attn_inputs(7, (1, ATTN["H"], T, ATTN["D"])))
        q, k, v = (x[:, u0:u0 + un].contiguous() for x in (q, k, v))
        sk = torch.zeros(un, device=dev)
        o = torch.empty_like(q)
        fn = lambda i: A.flash_attention(q, k, v, sk, kind="asinh", n=ATTN["n"], c=ATTN["c"], range_guard=True,  # noqa: E731
                                         shift=False, impl=args.kernel, out=o)
        for i in range(2):
            fn(i)
        ms_p = max_over_ranks(cuda_time(fn, max(3, min(args.steps, 10)), sync))
        part[f"seq{T}"] = {"ms": ms_p, "tflops_total": attn_flops(1, ATTN["H"], T, ATTN["D"]) / (ms_p * 1e-3) / 1e12,
                           "heads_per_gpu": un}
        del q, k, v, o
    extra["attn_heads_partitioned"] = dict(part, note="16 heads of config 5 dealt over the ranks, guarded call, max over ranks")
    torch.cuda.empty_cache()

    # ---- full prefill forward (benchmark configurations 3 and 4): batch split over ranks, hidden
    #      states all-gathered, head vocabulary-sharded ----
    from algebraic_transformer_b200 import prefill as PF
    # (name, model, vocab, batch, seq, weak): the configurations' batch is taken as the GLOBAL batch and
    # split over the ranks (strong scaling).  At N > 1 one more line gives every rank the whole batch of
    # the 125M configuration (weak scaling), the other reading of "scales from 1 to 8 GPUs".
    runs = [("prefill_125m", "125m", 50304, 16, 1024, False), ("prefill_350m", "350m", 32000, 8, 2048, False),
            ("prefill_1b", "1b", 32000, 8, 2048, False)]
    if world > 1:
        runs.append(("prefill_125m_weak", "125m", 50304, 16 * world, 1024, True))
    for name, size, vocab, gb, seq, weak in runs:
        if gb % world or (args.prefill_only is not None and args.prefill_only != size):
            continue
        cfg = PF.PrefillConfig.preset(size, vocab_size=vocab)
        params = PF.init_params(cfg, seed=0)
        ex = None
        if world > 1:
            try:
                from algebraic_transformer_b200.dist import HeadExchange
                ex = HeadExchange(dist.group.WORLD, gb * seq, dev)
            except Exception:
                ex = None                               # fall back to the NCCL all-reduce
        model = PF.Prefill(cfg, params, dev, seq_len=seq, impl=args.kernel, exchange=ex)
        del params
        gt = torch.Generator().manual_seed(2)
        tokens = torch.randint(0, vocab, (gb, seq), generator=gt)
        lb = gb // world
        tok = tokens[rank * lb:(rank + 1) * lb].to(dev)
        group = dist.group.WORLD if world > 1 else None

        replay, outputs, how = model.graphed_loss(tok, tok, group=group, rank=rank, world=world)

        def prefill_step(i):
            replay()

        for i in range(3):
            prefill_step(i)
        ms_p = max_over_ranks(cuda_time(prefill_step, max(3, min(args.steps, 10)), sync))
        fl = cfg.flops_per_token(seq) * gb * seq
        extra[name] = {"workload": f"{size}, global batch {gb} x {seq}, vocab {vocab}, batch split x{world}" + (" (weak)" if weak else ""),
                       "tokens_per_s": gb * seq / (ms_p * 1e-3), "ms_per_step": ms_p, "launch": how,
                       "head_exchange": "fused peer-memory kernel" if ex is not None else ("NCCL all-reduce" if world > 1 else "none"),
                       "tflops": fl / (ms_p * 1e-3) / 1e12, "frac_of_bf16_peak_per_gpu": fl / (ms_p * 1e-3) / 1e12 / world / peak_tf}
        if world > 1 and name == "prefill_125m":
            # the sharded objective against the same batch on one rank (no gather, no exchange)
            obj_sharded = float(model.loss(tok, tok, group=group, rank=rank, world=world)[0])
            if rank == 0:
                solo = PF.Prefill(cfg, PF.init_params(cfg, seed=0), dev, seq_len=seq, impl=args.kernel)
                all_tok = tokens.to(dev)
                obj_single = float(solo.loss(all_tok, all_tok)[0])
                parity["prefill_125m_objective_rel_diff"] = abs(obj_sharded - obj_single) / abs(obj_single)
                del solo, all_tok
        del replay, outputs, model, ex
        torch.cuda.empty_cache()
    if world > 1:
        extra["parity_multi_gpu"] = parity
        return extra, roofline_head

    # ---- configuration 5 at the longer sequences: the kernel alone and the guarded call ----
    for T in (16384, 32768):
        q, k, v = (x.to(dev) for x in make_attn_inputs(11, (1, ATTN["H"], T, ATTN["D"])))
        sk = torch.zeros(ATTN["H"], device=dev)
        o = torch.empty_like(q)
        f_k = lambda i: A.ops._attention_unshifted_unclamped(q, k, v, sk, n=ATTN["n"], c=ATTN["c"], impl=args.kernel, out=o)  # noqa: E731
        f_g = lambda i: A.flash_attention(q, k, v, sk, kind="asinh", n=ATTN["n"], c=ATTN["c"], range_guard=True, shift=False,  # noqa: E731
                                          impl=args.kernel, out=o)
        n_it = 5 if T == 16384 else 3
        for i in range(2):
            f_k(i)
        ms_k = cuda_time(f_k, n_it, sync)
        for i in range(2):
            f_g(i)
        ms_g = cuda_time(f_g, n_it, sync)
        fl = attn_flops(1, ATTN["H"], T, ATTN["D"])
        extra[f"attn_seq{T}"] = {"kernel_ms": ms_k, "kernel_frac_of_bf16_peak": fl / (ms_k * 1e-3) / 1e12 / peak_tf,
                                 "guarded_call_ms": ms_g, "guarded_call_frac_of_bf16_peak": fl / (ms_g * 1e-3) / 1e12 / peak_tf}
        del q, k, v, o
    # the max-shifted form on the same kernel (what a failed guard costs): explicit shift=True at 8192
    q, k, v = (x.to(dev) for x in make_attn_inputs(12, (1, ATTN["H"], ATTN["T"], ATTN["D"])))
    sk = torch.zeros(ATTN["H"], device=dev)
    o = torch.empty_like(q)
    f_s = lambda i: A.flash_attention(q, k, v, sk, kind="asinh", n=ATTN["n"], c=ATTN["c"], shift=True, impl=args.kernel, out=o)  # noqa: E731
    f_u = lambda i: A.ops._attention_unshifted_unclamped(q, k, v, sk, n=ATTN["n"], c=ATTN["c"], impl=args.kernel, out=o)  # noqa: E731
    for i in range(3):
        f_s(i)
    ms_s = cuda_time(f_s, iters, sync)
    for i in range(3):
        f_u(i)
    ms_u = cuda_time(f_u, iters, sync)
    fl = attn_flops(1, ATTN["H"], ATTN["T"], ATTN["D"])
    extra["attn_shifted_seq8192"] = {"ms": ms_s, "frac_of_bf16_peak": fl / (ms_s * 1e-3) / 1e12 / peak_tf,
                                     "unshifted_ms_same_inputs": ms_u, "ratio": ms_s / ms_u}
    del q, k, v, o
    # configuration 1 on the GPU: (4,12,1024,64) fp32, QK-norm + rotation prologue, guarded call; the tcgen05
    # kernel on bf16 hi | lo halves against the mma.sync kernel on the same inputs
    shape1 = (4, 12, 1024, 64)
    g1 = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(shape1, generator=g1).to(dev) for _ in range(3))
    sk = (torch.randn(shape1[1], generator=g1) * 0.02).to(dev)
    gain1 = torch.ones(shape1[3], device=dev)
    cos1, sin1 = A.cayley_table_geometric(shape1[3], shape1[2], device=dev)
    o = torch.empty_like(q)
    line = {"shape": list(shape1), "dtype": "f32", "flop_convention": "bf16-equivalent 4 B H T^2 D / 2 (each product is issued three times)"}
    for which in ("auto", "mma"):
        f_1 = lambda i: A.flash_attention(q, k, v, sk, kind="asinh", n=16, c=8.0, range_guard=True, q_gain=gain1, k_gain=gain1,  # noqa: E731
                                          cos=cos1, sin=sin1, impl=which, out=o)
        for i in range(3):
            f_1(i)
        ms_1 = cuda_time(f_1, iters, sync)
        line["ms" if which == "auto" else "ms_mma_sync"] = ms_1
        line["tflops" if which == "auto" else "tflops_mma_sync"] = attn_flops(*shape1) / (ms_1 * 1e-3) / 1e12
    extra["attn_config1_fp32"] = line
    del q, k, v, o
    # the attention shapes inside the prefill models (head_dim 64)
    for name, shape in (("attn_125m_layer", (16, 12, 1024, 64)), ("attn_350m_layer", (8, 16, 2048, 64))):
        q, k, v = (x.to(dev) for x in make_attn_inputs(13, shape))
        sk = torch.zeros(shape[1], device=dev)
        o = torch.empty_like(q)
        f_k = lambda i: A.ops._attention_unshifted_unclamped(q, k, v, sk, n=16, c=8.0, impl=args.kernel, out=o)  # noqa: E731
        for i in range(3):
            f_k(i)
        ms_k = cuda_time(f_k, iters, sync)
        extra[name] = {"shape": list(shape), "kernel_ms": ms_k, "tflops": attn_flops(*shape) / (ms_k * 1e-3) / 1e12,
                       "frac_of_bf16_peak": attn_flops(*shape) / (ms_k * 1e-3) / 1e12 / peak_tf}
        del q, k, v, o
    torch.cuda.empty_cache()
    # ---- standalone qk_rms (+ rotation): HBM bound ----
    B, H, T, D = 1, 16, 32768, 128
    x = torch.randn((B, H, T, D), generator=g).bfloat16().to(dev)
    y = torch.empty_like(x)
    gain = torch.ones(D, device=dev)
    cos, sin = A.cayley_table_geometric(D, T, device=dev)
    for rot in (False, True):
        kw = dict(cos=cos, sin=sin) if rot else {}
        fn = lambda i: A.qk_rms_norm(x, gain, out=y, **kw)  # noqa: E731
        for i in range(3):
            fn(i)
        ms_r = cuda_time(fn, iters, sync)
        # rows in and out; the rotated form also reads each position's fp32 cos/sin table rows once
        nbytes = 2.0 * x.numel() * 2 + ((cos.numel() + sin.numel()) * 4 if rot else 0)
        extra["qk_rms_rot" if rot else "qk_rms"] = {
            "workload": f"(1,16,{T},{D}) bf16, 134 MB in + out" + (", 17 MB of fp32 rotation tables in" if rot else ""),
            "ms": ms_r,
            "gbs": nbytes / (ms_r * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms_r * 1e-3) / 1e9 / peak_bw}
    # backward of the same normalisation: reads x and dy, writes dx (+ the gain gradient)
    fnb = lambda i: A.ops.qk_rms_norm_backward(x, gain, y, 1e-5)  # noqa: E731
    for i in range(3):
        fnb(i)
    ms_rb = cuda_time(fnb, iters, sync)
    nbytes_b = 3.0 * x.numel() * 2
    extra["qk_rms_bwd"] = {"workload": "x, dy in, dx out (3 x 134 MB) + dgain", "ms": ms_rb,
                           "gbs": nbytes_b / (ms_rb * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes_b / (ms_rb * 1e-3) / 1e9 / peak_bw}
    # ---- single-query decode against a 32768-token KV cache: HBM bound ----
    k = x
    v = torch.randn((B, H, T, D), generator=g).bfloat16().to(dev)
    qd = torch.randn((B, H, 1, D), generator=g).bfloat16().to(dev)
    od = torch.empty((B, H, 1, D), dtype=torch.bfloat16, device=dev)
    sink = torch.zeros(H, device=dev)
    fn = lambda i: A.decode_attention(qd, k, v, sink, n=16, c=8.0, out=od)  # noqa: E731
    for i in range(3):
        fn(i)
    # 268 MB of K,V > L2, so back-to-back launches already stream from HBM
    ms_d = cuda_time(fn, iters, sync)
    nbytes = 2.0 * k.numel() * 2
    extra["decode"] = {"workload": f"Tq=1 vs KV cache (1,16,{T},{D}) bf16, 268 MB", "ms": ms_d,
                       "gbs": nbytes / (ms_d * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms_d * 1e-3) / 1e9 / peak_bw}
    del k, v, x, y
    # ---- the two fused projections of one 125M block (16384 tokens): tensor bound ----
    M, dm, Hh, Dh, ff, Tt = 16384, 768, 12, 64, 2048, 1024
    xs = torch.randn((M, dm), generator=g).bfloat16().to(dev)
    wqkv = (torch.randn((3 * dm, dm), generator=g) * 0.05).bfloat16().to(dev)
    wgu = (torch.randn((2 * ff, dm), generator=g) * 0.05).bfloat16().to(dev)
    c2, s2 = A.cayley_table_geometric(Dh, Tt, device=dev)
    c2, s2 = c2.bfloat16().contiguous(), s2.bfloat16().contiguous()
    ones = torch.ones(Dh, device=dev)
    words = torch.zeros(4, dtype=torch.int32, device=dev)
    o_qkv = torch.empty((M, 3 * dm), dtype=torch.bfloat16, device=dev)
    o_glu = torch.empty((M, ff), dtype=torch.bfloat16, device=dev)
    for name, fn, fl in (
            ("qkv_proj_125m", lambda i: A.qkv_projection(xs, wqkv, Hh, Tt, c2, s2, ones, ones, 1e-5, 8.0, words, out=o_qkv),
             2.0 * M * dm * 3 * dm),
            ("glu_proj_125m", lambda i: A.glu_projection(xs, wgu, 0.5, out=o_glu), 2.0 * M * dm * 2 * ff)):
        for i in range(3):
            fn(i)
        ms_g = cuda_time(fn, iters, sync)
        extra[name] = {"workload": f"{M} tokens, d={dm}", "ms": ms_g, "tflops": fl / (ms_g * 1e-3) / 1e12,
                       "frac_of_bf16_peak": fl / (ms_g * 1e-3) / 1e12 / peak_tf}
    del xs, wqkv, wgu, o_qkv, o_glu
    # ---- attention backward (first "next" row): the 125M block's attention shape ----
    # and the headline attention shape; tcgen05 kernels ("auto") beside the mma.sync ones
    for name, (Bb, Hb, Tb, Db) in (("attn_bwd", (16, 12, 1024, 64)), ("attn_bwd_seq8192", (1, 16, 8192, 128))):
        qb_, kb_, vb_, dob_ = (torch.randn((Bb, Hb, Tb, Db), generator=g).bfloat16().to(dev) for _ in range(4))
        sk = torch.zeros(Hb, device=dev)
        ob_, stb_, kindb_ = A.flash_attention(qb_, kb_, vb_, sk, kind="asinh", n=16, c=8.0, range_guard=True, return_stat=True)
        flb = 2.5 * attn_flops(Bb, Hb, Tb, Db)
        row = {"shape": [Bb, Hb, Tb, Db], "flop_convention": "2.5 x forward"}
        for impl in ("auto", "mma"):
            fnb = lambda i: A.ops.flash_attention_backward(qb_, kb_, vb_, ob_, dob_, stb_, kindb_, sk, n=16, c=8.0, impl=impl)  # noqa: E731
            for i in range(3):
                fnb(i)
            ms_b = cuda_time(fnb, iters, sync)
            tag = "" if impl == "auto" else "_mma_sync"
            row["ms" + tag] = ms_b
            row["tflops" + tag] = flb / (ms_b * 1e-3) / 1e12
        row["frac_of_bf16_peak"] = row["tflops"] / peak_tf
        extra[name] = row
        del qb_, kb_, vb_, dob_, ob_, stb_
    # ---- Alg-CE head backward (second "next" row): configuration 2's shape ----
    Nh, dh_, Vh = HEAD["N"], HEAD["d"], HEAD["V"]
    hh = torch.randn((Nh, dh_), generator=g).bfloat16().to(dev)
    eh = (torch.randn((Vh, dh_), generator=g) * 0.02).bfloat16().to(dev)
    th = torch.randint(0, HEAD["target_hi"], (Nh,), generator=g).to(torch.int32).to(dev)
    sth = A.head_statistic(hh, eh, th, n=HEAD["n"], c=HEAD["c"])
    fnh = lambda i: A.ops.fused_head_backward(hh, eh, th, sth, n=HEAD["n"], c=HEAD["c"])  # noqa: E731
    for i in range(3):
        fnh(i)
    ms_hb = cuda_time(fnh, iters, sync)
    # the reference's control arm on the same kernel: softmax cross-entropy (online logsumexp epilogue)
    fnc = lambda i: A.head_statistic(hh, eh, th, kind="ce")  # noqa: E731
    for i in range(3):
        fnc(i)
    ms_ce = cuda_time(fnc, iters, sync)
    extra["ce_head"] = {"workload": "config 2 shape, kind='ce'", "ms": ms_ce, "tflops": 2.0 * Nh * dh_ * Vh / (ms_ce * 1e-3) / 1e12,
                        "frac_of_bf16_peak": 2.0 * Nh * dh_ * Vh / (ms_ce * 1e-3) / 1e12 / peak_tf}
    flh = 3 * 2.0 * Nh * dh_ * Vh                          # z again, dz . E, dz^T . h
    extra["alg_ce_head_bwd"] = {"workload": "config 2 shape: dz kernel + two cuBLAS GEMMs", "ms": ms_hb,
                                "tflops": flh / (ms_hb * 1e-3) / 1e12, "frac_of_bf16_peak": flh / (ms_hb * 1e-3) / 1e12 / peak_tf}
    return extra, roofline_head


if __name__ == "__main__":
    main()
