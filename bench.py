#!/usr/bin/env python
"""Benchmark of the quantized-KV decode-attention path (libnomos_attn.so, B200).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload at N=1 (configuration 2 of the baseline): one global-attention
decode layer, batch 1, 1 query token, 32 query / 16 KV heads, head_dim 128, 32768
cached keys, int8 per-token-per-head KV with fp32 scales, K with 4 outlier
channels per head (x8), bf16 Q, bf16 output.  A step is one pass of the hot path
(attention of the new query over the packed cache) for one layer.  At N GPUs the
job is N such sequences sharded by KV-head groups (16/N heads of every sequence
per GPU, no collective): per-GPU bytes are constant, i.e. weak scaling.

Metric: decode-attention HBM throughput = algorithmic bytes / time (GB/s), whole
job; us per layer is ms_per_step * 1000.  Inputs are synthetic, seeded, produced
on the device and quantised by the library's own quantize-on-write kernel.

One JSON line is printed on stdout by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "decode_attn_int8kv_32k_hbm_throughput"
UNIT = "GB/s"
NH, NKV, HD, T = 32, 16, 128, 32768
NLAYERS = 4                     # distinct layer caches cycled through, so no step finds its input in L2
SOFTMAX_SCALE = 1.0 / np.sqrt(128.0)


def algorithmic_bytes(nkv: int, kvg: int, t: int, hd: int, seqs: int = 1, s_rows: int = 1) -> int:
    """K+V payload + fp32 scales read once + bf16 Q read + bf16 output write."""
    return seqs * (2 * nkv * t * hd + 2 * nkv * t * 4 + s_rows * nkv * kvg * hd * (2 + 2))


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_peak_tflops() -> float:
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["bf16_tflops"])
    except Exception:
        return 1590.0


# --------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the GPU is busy."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.rows:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6 or not (t0 - 0.05 <= ts <= t1 + 0.15):
                continue
            try:
                sm.append(float(f[0])); mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------ workloads

def host_layer_rows(seed: int, nkv: int, t: int, hd: int):
    """One sequence's K and V rows of a layer, [t, nkv, hd] fp32: N(0,1) rounded to bf16, K with 4 outlier
    channels per head scaled x8 (configuration 2).  Seeded on the host, so the GPU arm and the CPU arm of the
    benchmark stream the same bytes once the rows are quantised (the library's quantize-on-write kernel and the
    oracle's are bit-identical)."""
    from oracle import oracle as orc
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((t, nkv, hd), dtype=np.float32)
    for h in range(nkv):
        k[:, h, rng.choice(hd, 4, replace=False)] *= np.float32(8.0)
    v = rng.standard_normal((t, nkv, hd), dtype=np.float32)
    return orc.bf16_round(k), orc.bf16_round(v)


def layer_seed(layer: int, rank: int, seq: int) -> int:
    return 1002 + 17 * layer + 1000 * rank + 100003 * seq


def workload_config(n: int) -> dict:
    """The `config` object of the JSON line; a function of the GPU count only, shared by both arms."""
    nkv_l = NKV // n
    by = algorithmic_bytes(nkv_l, NH // NKV, T, HD, n)
    return {"workload": f"C2 decode layer: {n} seq x 32768 cached keys, 32q/16kv heads x 128, int8 row-scale KV, "
                        f"bf16 Q/out, sharded by KV-head groups ({nkv_l} heads x {n} seq per GPU)",
            "bytes_per_step_per_gpu": by, "softmax_scale": "1/sqrt(128)",
            "l2": f"{NLAYERS} distinct layer caches cycled ({NLAYERS * by / 1e6:.0f} MB > 126 MB L2)",
            "seed": 1002, "flags": "NOMOS_ATTN_SETTLED_CACHE", "pdl_overlap": True,
            "launch_order": "attention launches back to back on one stream with programmatic dependent launch: the head "
                            "of launch i+1 (set-up, query preparation, first settled tiles) overlaps the tail of launch i"}


def make_layer_cache_from_host(torch, ops, dev, seqs: int, nkv: int, t: int, hd: int, layer: int, rank: int):
    """int8 cache [seqs, nkv, t, hd] + fp32 scales from host_layer_rows(), quantised on the device by the library's
    own quantize-on-write kernel.  Returns the device tensors."""
    k = torch.empty((seqs, nkv, t, hd), dtype=torch.int8, device=dev); v = torch.empty_like(k)
    ks = torch.empty((seqs, nkv, t), dtype=torch.float32, device=dev); vs = torch.empty_like(ks)
    chunk = 8192
    for s_ in range(seqs):
        hk, hv = host_layer_rows(layer_seed(layer, rank, s_), nkv, t, hd)
        for b in range(0, t, chunk):
            n = min(chunk, t - b)
            kk = torch.from_numpy(hk[b:b + n]).to(dev); vv = torch.from_numpy(hv[b:b + n]).to(dev)
            ops.gpu_append_quant_kv_i8(None, kk, vv, k[s_], v[s_], ks[s_], vs[s_], n, nkv, hd, nkv * hd, t, hd, b)
        torch.cuda.synchronize()
    return k, v, ks, vs


def host_quantised_layer(seed: int, nkv: int, t: int, hd: int):
    """The same layer quantised by the oracle on the host: (k int8 [nkv,t,hd], v, k_scales fp32 [nkv,t], v_scales)."""
    from oracle import oracle as orc
    hk, hv = host_layer_rows(seed, nkv, t, hd)
    k8 = np.zeros((nkv, t, hd), np.int8); v8 = np.zeros_like(k8)
    ks = np.zeros((nkv, t), np.float32); vs = np.zeros_like(ks)
    orc.append_quant_kv_i8(hk, hv, k8, v8, ks, vs, t, nkv, hd, nkv * hd, t, hd, 0)
    return k8, v8, ks, vs


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """max|got - want| / RMS(want): the quantity the parity tests gate at 2e-3."""
    w = want.astype(np.float64)
    return float(np.max(np.abs(got.astype(np.float64) - w)) / max(np.sqrt(np.mean(w * w)), 1e-30))


def make_layer_cache(torch, ops, dev, seqs: int, nkv: int, t: int, hd: int, seed: int):
    """int8 cache [seqs, nkv, t, hd] + fp32 scales, filled by the library's quantize-on-write
    kernel from seeded N(0,1) bf16 values (K: 4 outlier channels per head x8)."""
    g = torch.Generator(device=dev); g.manual_seed(seed)
    k = torch.empty((seqs, nkv, t, hd), dtype=torch.int8, device=dev); v = torch.empty_like(k)
    ks = torch.empty((seqs, nkv, t), dtype=torch.float32, device=dev); vs = torch.empty_like(ks)
    chunk = 4096
    for s in range(seqs):
        gain = torch.ones((nkv, hd), device=dev)
        for h in range(nkv):
            idx = torch.randperm(hd, generator=g, device=dev)[:4]
            gain[h, idx] = 8.0
        for b in range(0, t, chunk):
            n = min(chunk, t - b)
            kk = torch.randn((n, nkv, hd), generator=g, device=dev).to(torch.bfloat16).float() * gain
            kk = kk.to(torch.bfloat16).float().contiguous()
            vv = torch.randn((n, nkv, hd), generator=g, device=dev).to(torch.bfloat16).float().contiguous()
            ops.gpu_append_quant_kv_i8(None, kk, vv, k[s], v[s], ks[s], vs[s], n, nkv, hd, nkv * hd, t, hd, b)
    torch.cuda.synchronize()
    return k, v, ks, vs


def decode_args(ops, q, cache, out, nh, nkv, hd, t, seqs, **kw):
    k, v, ks, vs = cache
    return ops.make_args(q=q, k_cache=k, v_cache=v, k_scales=ks, v_scales=vs, out=out, kv_fmt=ops.KV_I8,
                         q_type=ops.BF16, out_type=ops.BF16, batch=seqs, nh=nh, nkv=nkv, kvg=nh // nkv, l_hd=hd,
                         cache_hd=hd, cache_cap=t, klen=t, softmax_scale=SOFTMAX_SCALE,
                         flags=ops.SETTLED_CACHE, **kw)   # decode loop: only the newest row is written per step


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from nomos_nvfp4_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    N = world
    from nomos_nvfp4_b200.sharding import head_group_shard
    shard = head_group_shard(NKV, NH // NKV, N, rank)      # this rank: its KV-head group of each of N sequences
    nkv_l, nh_l, seqs = shard.nkv, shard.nh, N
    step_bytes_rank = algorithmic_bytes(nkv_l, NH // NKV, T, HD, seqs)

    caches = [make_layer_cache_from_host(torch, ops, dev, seqs, nkv_l, T, HD, i, rank) for i in range(NLAYERS)]
    qrng = np.random.default_rng(2002 + rank)
    qs_host = [qrng.standard_normal((seqs, 1, nh_l, HD), dtype=np.float32) for _ in range(NLAYERS)]
    qs = [torch.from_numpy(x).to(dev).to(torch.bfloat16) for x in qs_host]
    outs = [torch.zeros((seqs, 1, nh_l, HD), dtype=torch.bfloat16, device=dev) for _ in range(NLAYERS)]
    a0 = decode_args(ops, qs[0], caches[0], outs[0], nh_l, nkv_l, HD, T, seqs)
    ws_bytes = ops.attn_workspace_bytes(a0)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    layer_args = [decode_args(ops, qs[i], caches[i], outs[i], nh_l, nkv_l, HD, T, seqs, workspace=ws, ws_bytes=ws_bytes)
                  for i in range(NLAYERS)]
    launches_per_step = 1               # one fused kernel per layer call (the split merge runs inside it)
    stream = torch.cuda.current_stream().cuda_stream

    def step(i):
        ops.attn_fused(stream, layer_args[i % NLAYERS])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(max(args.warmup, 3)):
        step(i)
    # keep the GPU busy long enough for the clock sampler to see it under load (untimed)
    t_busy = time.time()
    while not args.quick and time.time() - t_busy < 0.6:
        for i in range(200):
            step(i)
        torch.cuda.synchronize()
    barrier()
    t0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    t1 = time.time()
    ms = e0.elapsed_time(e1)
    if world > 1:
        tt = torch.tensor([ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    ms_per_step = ms / args.steps
    value = N * step_bytes_rank / (ms_per_step * 1e-3) / 1e9

    # per-launch duration of the hot path (attention kernel + split merge), one event pair per step
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(min(args.steps, 200))]
    for i, (a, b) in enumerate(evs):
        a.record(); step(i); b.record()
    torch.cuda.synchronize()
    per = sorted(a.elapsed_time(b) for a, b in evs)
    kern_ms = float(np.mean(per))
    clocks = sampler.stop(t_busy, time.time()) if rank == 0 else None

    # Parity of what was timed: layer 0's attention (the timed call with an fp32 output buffer) against the oracle's
    # exact attention over the same cache bytes, quantised on the host from the same seeded rows; sequence 0 of rank 0.
    # Done here, before the end-to-end legs append rows to the caches.
    parity = None
    if rank == 0 and not args.no_parity and not args.quick:
        from oracle import oracle as orc
        k8, v8, ks8, vs8 = host_quantised_layer(layer_seed(0, rank, 0), nkv_l, T, HD)
        same_bytes = bool(np.array_equal(caches[0][0][0].cpu().numpy(), k8) and np.array_equal(caches[0][2][0].cpu().numpy(), ks8)
                          and np.array_equal(caches[0][1][0].cpu().numpy(), v8) and np.array_equal(caches[0][3][0].cpu().numpy(), vs8))
        out32 = torch.zeros((seqs, 1, nh_l, HD), dtype=torch.float32, device=dev)
        a32 = decode_args(ops, qs[0], caches[0], out32, nh_l, nkv_l, HD, T, seqs, workspace=ws, ws_bytes=ws_bytes)
        a32.out_type = ops.F32
        ops.attn_fused(stream, a32); torch.cuda.synchronize()
        want = orc.attn_exact(orc.bf16_round(qs_host[0][0]), k8, v8, ks8, vs8, orc.KV_I8, nh_l, nkv_l, HD, HD, T,
                              query_base_pos=T - 1, softmax_scale=float(SOFTMAX_SCALE))
        parity = {"value": float(f"{rel_err(out32[0].cpu().numpy(), want):.3e}"), "bar": 2e-3,
                  "what": "max|out - exact| / RMS(exact), fp32 output of the timed call (layer 0, sequence 0) against the oracle's "
                          "fp64 attention over the same cache bytes", "cache_bytes_equal_oracle": same_bytes}

    if args.quick:      # profiling mode: only the warm-up and the timed steps ran
        if world > 1:
            dist.destroy_process_group()
        return {"metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": N, "steps": args.steps,
                "ms_per_step": round(ms_per_step, 6), "quick": True} if rank == 0 else {}

    # end to end through the C ABI with HOST buffers (nomos_attn_fused_host): per step the bf16 query and the new
    # token's fp32 K/V rows come from pinned host memory (h2d bytes), the fused kernel appends and attends, the bf16
    # output lands in pinned host memory (d2h bytes), the host synchronises -- all inside ONE library call.  The
    # inputs are staged by a small copy kernel (the attention grid is set up behind it); the kernel writes its result into the pinned output buffer itself.
    q_bytes, kv_bytes = seqs * nh_l * HD * 2, seqs * nkv_l * HD * 4
    stage_h = torch.empty(q_bytes + 2 * kv_bytes, dtype=torch.uint8).pin_memory()
    stage_h[:q_bytes].view(torch.bfloat16).copy_(torch.randn(seqs * nh_l * HD).to(torch.bfloat16))
    stage_h[q_bytes:].view(torch.float32).copy_(torch.randn(2 * seqs * nkv_l * HD))
    stage_d = torch.empty_like(stage_h, device=dev)
    host_out = torch.empty((seqs, 1, nh_l, HD), dtype=torch.bfloat16).pin_memory()
    e2e_args = []
    for i in range(NLAYERS):
        k, v, ks, vs = caches[i]
        e2e_args.append(ops.make_args(
            q=stage_d.data_ptr(), k_cache=k, v_cache=v, k_scales=ks, v_scales=vs, out=outs[i], kv_fmt=ops.KV_I8,
            q_type=ops.BF16, out_type=ops.BF16, batch=seqs, nh=nh_l, nkv=nkv_l, kvg=nh_l // nkv_l, l_hd=HD, cache_hd=HD,
            cache_cap=T, klen=T, softmax_scale=SOFTMAX_SCALE, flags=ops.SETTLED_CACHE, workspace=ws, ws_bytes=ws_bytes,
            new_k=stage_d.data_ptr() + q_bytes, new_v=stage_d.data_ptr() + q_bytes + kv_bytes, n_new=1, new_base_pos=T - 1))
    h2d, d2h = stage_h.numel(), host_out.numel() * 2

    hin, din, hout = stage_h.data_ptr(), stage_d.data_ptr(), host_out.data_ptr()
    douts = [o.data_ptr() for o in outs]

    def e2e_step(i):
        # nomos_attn_fused_host: staging kernel H2D, the fused kernel (writing the pinned output itself), cudaStreamSynchronize
        j = i % NLAYERS
        ops.attn_fused_host(stream, e2e_args[j], hin, din, h2d, hout, douts[j], d2h)

    for i in range(3):
        e2e_step(i)
    barrier()
    n_e2e = min(args.steps, 200)
    tw0 = time.perf_counter()
    for i in range(n_e2e):
        e2e_step(i)
    tw1 = time.perf_counter()
    e2e_s = (tw1 - tw0) / n_e2e
    if world > 1:
        tt = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = float(tt.item())
    e2e_val = N * step_bytes_rank / e2e_s / 1e9

    # variant: the same step with explicit runtime copies around the device-buffer call (what nomos_attn_fused_host
    # does for pageable or large host buffers): cudaMemcpyAsync H2D, nomos_attn_fused, cudaMemcpyAsync D2H, synchronise
    def copy_step(i):
        j = i % NLAYERS
        stage_d.copy_(stage_h, non_blocking=True)
        ops.attn_fused(stream, e2e_args[j])
        host_out.copy_(outs[j], non_blocking=True)
        torch.cuda.synchronize()

    for i in range(3):
        copy_step(i)
    barrier()
    tw0 = time.perf_counter()
    for i in range(n_e2e):
        copy_step(i)
    zc_s = (time.perf_counter() - tw0) / n_e2e
    if world > 1:
        tt = torch.tensor([zc_s], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        zc_s = float(tt.item())

    peak, peak_src = measured_peak_gbs()
    tc5 = ops.attn_kernel_choice(layer_args[0]) == 1          # which of the two kernels the library runs for this call
    kernel_name = ("attn_tc5_kernel<2> (tcgen05 + TMEM + TMA)" if tc5
                   else "attn_fused_kernel<int8,128,1> (int8 mma.sync + TMA tiles + mbarrier ring)")
    # roofline: algorithmic bytes / average launch duration over the timed region (launches run
    # back to back there, as they do in a decode loop); the event-bracketed single launch is kept too
    achieved = step_bytes_rank / (ms_per_step * 1e-3) / 1e9
    result = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": N, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 6), "us_per_layer": round(ms_per_step * 1000, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": ("int8 (KV bytes x fixed-point Q / softmax weights on tcgen05 int8 tensor cores, int32 in tensor memory, fp32 running sums)" if tc5
                                                          else "int8 (KV bytes x fixed-point Q / softmax weights on int8 tensor cores, int32 accumulators, fp32 running sums)"),
        "data": "synthetic",
        "config": workload_config(N),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": None, "peak_source": f"of {peak_src}",
                     "kernel": kernel_name, "launch_us": round(ms_per_step * 1000, 3),
                     "launch_us_isolated": round(kern_ms * 1000, 3),
                     "frac_isolated": round(step_bytes_rank / (kern_ms * 1e-3) / 1e9 / peak, 4),
                     "note": "frac: average over the timed region, where consecutive launches overlap head to tail "
                             "(programmatic dependent launch); frac_isolated: one launch bracketed by its own events"},
        "e2e": {"value": round(e2e_val, 1), "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "us_per_layer": round(e2e_s * 1e6, 2),
                "path": "nomos_attn_fused_host: inputs staged from pinned host memory by a copy kernel the attention grid is chained behind, output written to pinned host memory by the attention kernel, stream synchronised",
                "explicit_copies_us_per_layer": round(zc_s * 1e6, 2)},
        "gpu_launches": int(args.steps * launches_per_step),
        "clocks": clocks,
    }
    # dram__bytes_read.sum + dram__bytes_write.sum per launch.  ncu captured one launch of each kernel on exactly the
    # N=1 workload (138,428,416 algorithmic bytes): 143.48 MB for the tcgen05 kernel, 142.00 MB for the mma.sync
    # kernel.  The traffic is the streamed cache plus the split partials, both proportional to the bytes a launch
    # processes, so other per-GPU workloads scale the captured figure by their algorithmic bytes.
    result["roofline"]["traffic"] = round((143.48e6 if tc5 else 142.00e6) * step_bytes_rank / 138428416.0)

    if parity is not None:
        result["parity_rel_err"] = parity

    if rank == 0 and N == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_reference_leg()
    if not args.no_extras:
        result["extras"] = extras(torch, dist, ops, dev, rank, world)
        # the two long-context curves of configuration 5 at the top level: c5a has no collective (KV-head groups),
        # c5b exchanges (o, m, l) between the ranks inside the timed step (strong scaling: the job is fixed)
        for key, name in (("c5a_batch8_131k_head_sharded", "c5a"), ("c5b_seq_sharded_512k", "c5b")):
            e = result["extras"].get(key, {})
            if "us_per_layer" in e:
                result[name] = {"us_per_layer": e["us_per_layer"], "n_gpus": N, "scaling": "strong",
                                "GBps_aggregate": e.get("GBps_aggregate")}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result if rank == 0 else {}


# -------------------------------------------------------------------- extras

def time_call(torch, fn, iters: int, warm: int = 5) -> float:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1000.0       # us


def extras(torch, dist, ops, dev, rank, world, iters: int = 200, only=None) -> dict:
    """Secondary configurations, bounded in time.  Not the headline; reported for context.
    `only`: names of the cases to run (profiler captures run one case by itself)."""
    out = {}

    def selected(*names):
        return only is None or any(n in only for n in names)
    stream = torch.cuda.current_stream().cuda_stream
    # configuration 4: verify, VB = 9 rows against 16384 cached keys (+9 new), int8 KV.
    # Four layer caches are cycled (278 MB > L2), as a 60-layer verify pass would.
    if selected("c4_verify_vb9_16k"):
        try:
            S, T4 = 9, 16384 + 9
            caches = [make_layer_cache(torch, ops, dev, 1, NKV, T4, HD, 1004 + i) for i in range(NLAYERS)]
            q = torch.from_numpy(np.random.default_rng(4004 + rank).standard_normal((1, S, NH, HD), dtype=np.float32)).to(dev).to(torch.bfloat16)
            o = torch.zeros((1, S, NH, HD), dtype=torch.bfloat16, device=dev)
            al = []
            for k, v, ks, vs in caches:
                al.append(ops.make_args(q=q, k_cache=k, v_cache=v, k_scales=ks, v_scales=vs, out=o, kv_fmt=ops.KV_I8,
                                        q_type=ops.BF16, out_type=ops.BF16, S=S, nh=NH, nkv=NKV, kvg=NH // NKV, l_hd=HD,
                                        cache_hd=HD, cache_cap=T4, klen=T4, softmax_scale=SOFTMAX_SCALE))
            wsb = ops.attn_workspace_bytes(al[0])
            ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
            for a in al:
                a.workspace, a.ws_bytes = ws.data_ptr(), wsb
            ctr = [0]

            def fn4():
                ops.attn_fused(stream, al[ctr[0] % NLAYERS]); ctr[0] += 1

            us = time_call(torch, fn4, iters)
            by = algorithmic_bytes(NKV, NH // NKV, T4, HD, 1, S)
            out["c4_verify_vb9_16k"] = {"us_per_layer": round(us, 2), "GBps": round(by / us / 1e3, 1),
                                        "attn_only_tok_per_s_60_layers": round(S / (60 * us * 1e-6), 1)}
            if rank == 0:          # parity of the timed call (fp32 output, layer 0) against the oracle, every row against its own RMS
                from oracle import oracle as orc
                o32 = torch.zeros((1, S, NH, HD), dtype=torch.float32, device=dev)
                al[0].out, al[0].out_type = o32.data_ptr(), ops.F32
                ops.attn_fused(stream, al[0]); torch.cuda.synchronize()
                k0, v0, ks0, vs0 = (t[0].cpu().numpy() for t in caches[0])
                want = orc.attn_exact(q[0].float().cpu().numpy(), k0, v0, ks0, vs0, orc.KV_I8, NH, NKV, HD, HD, T4, S=S,
                                      query_base_pos=T4 - S, softmax_scale=float(SOFTMAX_SCALE))
                got = o32[0].cpu().numpy()
                out["c4_verify_vb9_16k"]["parity_rel_err"] = float(f"{max(rel_err(got[r], want[r]) for r in range(S)):.3e}")
            del caches, ws
        except Exception as e:   # report, never hide
            out["c4_verify_vb9_16k"] = {"error": str(e)}
    # prefill: 2048 prompt tokens, 32q/16kv x 128, int8 KV already appended; causal attention over the quantised
    # cache on the query-major tcgen05 kernel (no S x S score matrix), and the same call as mma.sync row groups
    if selected("prefill_s2048_i8"):
        try:
            Sp = 2048
            cache = make_layer_cache(torch, ops, dev, 1, NKV, Sp, HD, 1404)
            qh = np.random.default_rng(1404).standard_normal((1, Sp, NH, HD), dtype=np.float32)
            q = torch.from_numpy(qh).to(dev).to(torch.bfloat16)
            o = torch.zeros((1, Sp, NH, HD), dtype=torch.bfloat16, device=dev)
            k, v, ks, vs = cache
            res = {}
            for name, fl in (("tcgen05_query_major", 0), ("mma_sync_row_groups", ops.NO_TCGEN05)):
                a = ops.make_args(q=q, k_cache=k, v_cache=v, k_scales=ks, v_scales=vs, out=o, kv_fmt=ops.KV_I8, q_type=ops.BF16,
                                  out_type=ops.BF16, S=Sp, nh=NH, nkv=NKV, kvg=NH // NKV, l_hd=HD, cache_hd=HD, cache_cap=Sp, klen=Sp,
                                  softmax_scale=SOFTMAX_SCALE, flags=fl)
                wsb = ops.attn_workspace_bytes(a)
                ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
                a.workspace, a.ws_bytes = ws.data_ptr(), wsb
                us = time_call(torch, lambda: ops.attn_fused(stream, a), max(10, iters // 8))
                flops = 4.0 * NH * HD * (Sp * (Sp + 1) / 2.0)           # QK and PV over the causal half
                res[name] = {"us": round(us, 1), "TFLOPs_causal": round(flops / us / 1e6, 1), "kernel_choice": ops.attn_kernel_choice(a)}
                if rank == 0 and fl == 0:
                    from oracle import oracle as orc
                    o32 = torch.zeros((1, Sp, NH, HD), dtype=torch.float32, device=dev)
                    a.out, a.out_type = o32.data_ptr(), ops.F32
                    ops.attn_fused(stream, a); torch.cuda.synchronize()
                    a.out, a.out_type = o.data_ptr(), ops.BF16
                    got = o32[0].cpu().numpy()
                    hk, hv, hks, hvs = (t[0].cpu().numpy() for t in cache)
                    worst = 0.0
                    for srow in (0, 1, 63, 64, 127, 128, 1000, 1023, 1024, 2047):
                        want = orc.attn_exact(orc.bf16_round(qh[0, srow:srow + 1]), hk, hv, hks, hvs, orc.KV_I8, NH, NKV, HD, HD, Sp, S=1,
                                              query_base_pos=srow, softmax_scale=float(SOFTMAX_SCALE))
                        worst = max(worst, rel_err(got[srow], want[0]))
                    res[name]["parity_rel_err_sampled_rows"] = float(f"{worst:.3e}")
            res["tensor_peak_fraction"] = round(res["tcgen05_query_major"]["TFLOPs_causal"] / measured_peak_tflops(), 4)
            out["prefill_s2048_i8"] = res
            del cache
        except Exception as e:
            out["prefill_s2048_i8"] = {"error": repr(e)}
    # chunked prefill: a chunk of 2048 new positions behind a cached prefix of 6144 (keys 0..8191 in the int8 cache),
    # the call an engine makes per prefill chunk (the reference's prefix operator, lib/attention_gpu_int8.mojo:844-887,
    # which needs a [nkv, S*kvg, 8192] score scratch for it); and one square prefill of 8192 positions
    if selected("prefill_chunk2048_prefix6144_i8"):
        try:
            Sp, Tp = 2048, 8192
            cache = make_layer_cache(torch, ops, dev, 1, NKV, Tp, HD, 1406)
            qh = np.random.default_rng(1406).standard_normal((1, Sp, NH, HD), dtype=np.float32)
            q = torch.from_numpy(qh).to(dev).to(torch.bfloat16)
            o = torch.zeros((1, Sp, NH, HD), dtype=torch.bfloat16, device=dev)
            k, v, ks, vs = cache
            a = ops.make_args(q=q, k_cache=k, v_cache=v, k_scales=ks, v_scales=vs, out=o, kv_fmt=ops.KV_I8, q_type=ops.BF16,
                              out_type=ops.BF16, S=Sp, nh=NH, nkv=NKV, kvg=NH // NKV, l_hd=HD, cache_hd=HD, cache_cap=Tp, klen=Tp,
                              softmax_scale=SOFTMAX_SCALE)
            wsb = ops.attn_workspace_bytes(a)
            ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
            a.workspace, a.ws_bytes = ws.data_ptr(), wsb
            us = time_call(torch, lambda: ops.attn_fused(stream, a), max(10, iters // 16))
            keys = sum(Tp - Sp + s + 1 for s in range(Sp))             # keys each query position attends
            flops = 4.0 * NH * HD * keys
            res = {"us": round(us, 1), "TFLOPs_causal": round(flops / us / 1e6, 1), "kernel_choice": ops.attn_kernel_choice(a),
                   "tensor_peak_fraction": round(flops / us / 1e6 / measured_peak_tflops(), 4)}
            if rank == 0:
                from oracle import oracle as orc
                o32 = torch.zeros((1, Sp, NH, HD), dtype=torch.float32, device=dev)
                a.out, a.out_type = o32.data_ptr(), ops.F32
                ops.attn_fused(stream, a); torch.cuda.synchronize()
                got = o32[0].cpu().numpy()
                hk, hv, hks, hvs = (t[0].cpu().numpy() for t in cache)
                worst = 0.0
                for srow in (0, 63, 64, 1000, 2047):
                    want = orc.attn_exact(orc.bf16_round(qh[0, srow:srow + 1]), hk, hv, hks, hvs, orc.KV_I8, NH, NKV, HD, HD, Tp, S=1,
                                          query_base_pos=Tp - Sp + srow, softmax_scale=float(SOFTMAX_SCALE))
                    worst = max(worst, rel_err(got[srow], want[0]))
                res["parity_rel_err_sampled_rows"] = float(f"{worst:.3e}")
            out["prefill_chunk2048_prefix6144_i8"] = res
            del cache, ws
        except Exception as e:
            out["prefill_chunk2048_prefix6144_i8"] = {"error": repr(e)}
    # configuration 3: sliding-window layer, ring of 1024 at position 8191, int4 block-32, fused append
    if selected("c3_swa_ring_i4b32_fused_append"):
        try:
            W, pos = 1024, 8191
            nb = HD // 32
            rows = NKV * W
            k = torch.zeros((NKV, W, HD // 2), dtype=torch.uint8, device=dev); v = torch.zeros_like(k)
            ks = torch.zeros(rows * nb * 2 + rows * 4, dtype=torch.uint8, device=dev); vs = torch.zeros_like(ks)
            g = torch.Generator(device=dev); g.manual_seed(1003)
            for base in range(0, pos, 1024):
                n = min(1024, pos - base)
                kk = torch.randn((n, NKV, HD), generator=g, device=dev).to(torch.bfloat16).float().contiguous()
                vv = torch.randn((n, NKV, HD), generator=g, device=dev).to(torch.bfloat16).float().contiguous()
                ops.gpu_append_quant_kv_i4(None, kk, vv, k, v, ks, vs, n, NKV, HD, NKV * HD, W, HD, base, nb)
            q = torch.randn((1, 1, NH, HD), device=dev).to(torch.bfloat16)
            o = torch.zeros((1, 1, NH, HD), dtype=torch.bfloat16, device=dev)
            nk = torch.randn((1, NKV, HD), device=dev); nv = torch.randn((1, NKV, HD), device=dev)
            a = ops.make_args(q=q, k_cache=k, v_cache=v, k_scales=ks, v_scales=vs, out=o, kv_fmt=ops.KV_I4B32, q_type=ops.BF16,
                              out_type=ops.BF16, nh=NH, nkv=NKV, kvg=NH // NKV, l_hd=HD, cache_hd=HD, cache_cap=W,
                              win_start=pos + 1 - W, klen=W, softmax_scale=SOFTMAX_SCALE, new_k=nk, new_v=nv, n_new=1,
                              new_base_pos=pos)
            wsb = ops.attn_workspace_bytes(a)
            ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
            a.workspace, a.ws_bytes = ws.data_ptr(), wsb
            us = time_call(torch, lambda: ops.attn_fused(stream, a), iters)
            out["c3_swa_ring_i4b32_fused_append"] = {"us_per_layer": round(us, 2), "bytes": 2394368,
                                                     "note": "2.4 MB per call: launch-latency-bound, L2-resident"}
        except Exception as e:
            out["c3_swa_ring_i4b32_fused_append"] = {"error": str(e)}
    # the reference model's real layer geometry (Gemma-4-31B, lib/gemma4_engine.mojo:371-392), int4 block-32 KV:
    # sliding layers 32q/16kv x 256 with a 1024-slot ring, full layers 32q/4kv x 512 at 32768 keys
    for name, nkv_g, hd_g, t_g, cap_g in (("g4_sliding_hd256_i4b32_w1024", 16, 256, 1024, 1024),
                                          ("g4_full_hd512_i4b32_32k", 4, 512, 32768, 32768)):
        if not selected(name):
            continue
        try:
            nb = hd_g // 32
            rows = nkv_g * cap_g
            cs = []
            for li in range(2 if t_g > 4096 else 1):
                k = torch.zeros((nkv_g, cap_g, hd_g // 2), dtype=torch.uint8, device=dev); v = torch.zeros_like(k)
                ks = torch.zeros(rows * nb * 2 + rows * 4, dtype=torch.uint8, device=dev); vs = torch.zeros_like(ks)
                g = torch.Generator(device=dev); g.manual_seed(77 + li)
                for base in range(0, t_g, 2048):
                    n = min(2048, t_g - base)
                    kk = torch.randn((n, nkv_g, hd_g), generator=g, device=dev).to(torch.bfloat16).float().contiguous()
                    vv = torch.randn((n, nkv_g, hd_g), generator=g, device=dev).to(torch.bfloat16).float().contiguous()
                    ops.gpu_append_quant_kv_i4(None, kk, vv, k, v, ks, vs, n, nkv_g, hd_g, nkv_g * hd_g, cap_g, hd_g, base, nb)
                cs.append((k, v, ks, vs))
            q = torch.randn((1, 1, NH, hd_g), device=dev).to(torch.bfloat16)
            o = torch.zeros((1, 1, NH, hd_g), dtype=torch.bfloat16, device=dev)
            al = [ops.make_args(q=q, k_cache=c[0], v_cache=c[1], k_scales=c[2], v_scales=c[3], out=o, kv_fmt=ops.KV_I4B32,
                                q_type=ops.BF16, out_type=ops.BF16, nh=NH, nkv=nkv_g, kvg=NH // nkv_g, l_hd=hd_g, cache_hd=hd_g,
                                cache_cap=cap_g, klen=t_g, softmax_scale=1.0 / np.sqrt(hd_g), flags=ops.SETTLED_CACHE) for c in cs]
            wsb = ops.attn_workspace_bytes(al[0])
            ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
            for a_ in al:
                a_.workspace, a_.ws_bytes = ws.data_ptr(), wsb
            cnt = [0]

            def fng():
                ops.attn_fused(stream, al[cnt[0] % len(al)]); cnt[0] += 1

            us = time_call(torch, fng, iters)
            by = 2 * nkv_g * t_g * (hd_g // 2) + 2 * nkv_g * t_g * nb * 2 + NH * hd_g * 4
            out[name] = {"us_per_layer": round(us, 2), "GBps": round(by / us / 1e3, 1), "bytes": by}
            del cs, ws
        except Exception as e:
            out[name] = {"error": str(e)}
    # producer epilogue: V-norm + QK-norm + RoPE + quantize-on-write of one decode token in one launch
    # (the reference: five kernels and the append), at the configurations' and the model's layer geometries
    for name, nh_p, nkv_p, hd_p, fmt_p, cap_p, theta_p, rdim_p in (
            ("producer_c2_hd128_i8", NH, NKV, HD, ops.KV_I8, 32768, 10000.0, HD),
            ("producer_g4_sliding_hd256_i4b32", NH, 16, 256, ops.KV_I4B32, 1024, 10000.0, 256),
            ("producer_g4_full_hd512_i4b32", NH, 4, 512, ops.KV_I4B32, 32768, 1000000.0, 128)):
        if not selected(name):
            continue
        try:
            row_b = hd_p if fmt_p == ops.KV_I8 else hd_p // 2
            nb = hd_p // 32
            sc_b = nkv_p * cap_p * (4 if fmt_p == ops.KV_I8 else nb * 2 + 4)
            ck = torch.zeros((nkv_p, cap_p, row_b), dtype=torch.uint8, device=dev); cv = torch.zeros_like(ck)
            cks = torch.zeros(sc_b, dtype=torch.uint8, device=dev); cvs = torch.zeros_like(cks)
            qp = torch.randn((1, nh_p, hd_p), device=dev); kp = torch.randn((1, nkv_p, hd_p), device=dev)
            vp = torch.randn((1, nkv_p, hd_p), device=dev)
            qw = torch.ones(hd_p, device=dev); kw = torch.ones(hd_p, device=dev)
            pos = [0]

            def fnp():
                ops.kv_norm_rope_append(stream, qp, qw, kp, vp, kw, ck, cv, cks, cvs, n_s=1, nh=nh_p, nkv=nkv_p, l_hd=hd_p,
                                        l_kvd=nkv_p * hd_p, cache_cap=cap_p, cache_hd=hd_p, base_pos=pos[0] % cap_p,
                                        theta=theta_p, rope_dim=rdim_p, kv_fmt=fmt_p)
                pos[0] += 1

            out[name] = {"us_per_call": round(time_call(torch, fnp, iters), 2), "launches": 1, "reference_launches": 6,
                         "note": "a few KB per call: bounded by the host's launch rate through ctypes, not by the GPU"}
            del ck, cv, cks, cvs
        except Exception as e:
            out[name] = {"error": str(e)}
    # one decode step of a layer's attention path at configuration 2: producer epilogue (norms, RoPE, quantize-on-write
    # of the new token) then attention over the 32768 keys -- two launches chained by programmatic dependent launch
    if selected("decode_step_c2_producer_plus_attention"):
        try:
            caches = [make_layer_cache(torch, ops, dev, 1, NKV, T, HD, 1302 + i) for i in range(NLAYERS)]
            qf = torch.randn((1, NH, HD), device=dev); kf = torch.randn((1, NKV, HD), device=dev); vf = torch.randn((1, NKV, HD), device=dev)
            qw = torch.ones(HD, device=dev); kw = torch.ones(HD, device=dev)
            o = torch.zeros((1, 1, NH, HD), dtype=torch.bfloat16, device=dev)
            al = []
            for k, v, ks, vs in caches:
                al.append((ops.make_args(q=qf, k_cache=k, v_cache=v, k_scales=ks, v_scales=vs, out=o, kv_fmt=ops.KV_I8, q_type=ops.F32,
                                         out_type=ops.BF16, nh=NH, nkv=NKV, kvg=NH // NKV, l_hd=HD, cache_hd=HD, cache_cap=T, klen=T,
                                         softmax_scale=SOFTMAX_SCALE, flags=ops.SETTLED_CACHE), (k, v, ks, vs)))
            wsb = ops.attn_workspace_bytes(al[0][0])
            ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
            for a_, _ in al:
                a_.workspace, a_.ws_bytes = ws.data_ptr(), wsb
            ctr2 = [0]

            def fstep():
                a_, (k, v, ks, vs) = al[ctr2[0] % NLAYERS]; ctr2[0] += 1
                ops.kv_norm_rope_append(stream, qf, qw, kf, vf, kw, k, v, ks, vs, n_s=1, nh=NH, nkv=NKV, l_hd=HD, l_kvd=NKV * HD,
                                        cache_cap=T, cache_hd=HD, base_pos=T - 1, theta=10000.0, rope_dim=HD, kv_fmt=ops.KV_I8)
                ops.attn_fused(stream, a_)

            us = time_call(torch, fstep, iters)
            out["decode_step_c2_producer_plus_attention"] = {"us_per_layer": round(us, 2), "launches": 2,
                                                             "reference_launches": "6 + append + 2 dequant + 5 attention"}
            del caches, ws
        except Exception as e:
            out["decode_step_c2_producer_plus_attention"] = {"error": str(e)}
    # configuration 5a: batch 8 x 131072 keys, sharded by KV-head groups (16 / world heads per GPU, no collective)
    if selected("c5a_batch8_131k_head_sharded"):
        try:
            B5, T5a = 8, 131072
            nkv5 = NKV // world
            nh5 = nkv5 * (NH // NKV)
            cache = make_layer_cache(torch, ops, dev, B5, nkv5, T5a, HD, 1105 + rank)
            q = torch.randn((B5, 1, nh5, HD), device=dev).to(torch.bfloat16)
            o = torch.zeros((B5, 1, nh5, HD), dtype=torch.bfloat16, device=dev)
            a5 = decode_args(ops, q, cache, o, nh5, nkv5, HD, T5a, B5)
            wsb = ops.attn_workspace_bytes(a5)
            ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
            a5.workspace, a5.ws_bytes = ws.data_ptr(), wsb
            us = time_call(torch, lambda: ops.attn_fused(stream, a5), max(10, iters // 8))
            if world > 1:
                tt = torch.tensor([us], device=dev); dist.all_reduce(tt, op=dist.ReduceOp.MAX); us = float(tt.item())
            by = algorithmic_bytes(NKV, NH // NKV, T5a, HD, B5)
            out["c5a_batch8_131k_head_sharded"] = {"us_per_layer": round(us, 2), "GBps_aggregate": round(by / us / 1e3, 1), "gpus": world}
            del cache, ws
        except Exception as e:
            out["c5a_batch8_131k_head_sharded"] = {"error": str(e)}
    # configuration 5a on PAGED caches: same bytes, pages of 128 keys behind a shuffled block table (serving layout)
    if selected("c5a_paged_batch8_131k"):
        try:
            B5, T5a = 8, 131072
            nkv5 = NKV // world
            nh5 = nkv5 * (NH // NKV)
            ppseq = T5a // 128
            n_pages = B5 * ppseq
            g = torch.Generator(device=dev); g.manual_seed(1205 + rank)
            kp = torch.randint(-127, 128, (n_pages, nkv5, 128, HD), dtype=torch.int8, device=dev, generator=g)
            vp = torch.randint(-127, 128, (n_pages, nkv5, 128, HD), dtype=torch.int8, device=dev, generator=g)
            ksp = torch.rand((n_pages, nkv5, 128), device=dev, generator=g) * 0.02 + 0.01
            vsp = torch.rand((n_pages, nkv5, 128), device=dev, generator=g) * 0.02 + 0.01
            table = torch.randperm(n_pages, device=dev, generator=g).to(torch.int32).reshape(B5, ppseq).contiguous()
            lens = torch.full((B5,), T5a, dtype=torch.int32, device=dev)
            q = torch.randn((B5, nh5, HD), device=dev).to(torch.bfloat16)
            o = torch.zeros((B5, nh5, HD), dtype=torch.bfloat16, device=dev)
            wsb = ops.attn_paged_workspace_bytes(B5, nh5, nkv5, NH // NKV, HD, T5a)
            ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)

            def fnpg():
                ops.attn_paged_decode_i8(stream, q, kp, vp, ksp, vsp, table, lens, o, ws, wsb, batch=B5, nh=nh5, nkv=nkv5, kvg=NH // NKV,
                                         l_hd=HD, n_pages=n_pages, max_pages=ppseq, max_len=T5a, softmax_scale=SOFTMAX_SCALE,
                                         q_type=ops.BF16, out_type=ops.BF16)

            us = time_call(torch, fnpg, max(10, iters // 8))
            if world > 1:
                tt = torch.tensor([us], device=dev); dist.all_reduce(tt, op=dist.ReduceOp.MAX); us = float(tt.item())
            by = algorithmic_bytes(NKV, NH // NKV, T5a, HD, B5)
            out["c5a_paged_batch8_131k"] = {"us_per_layer": round(us, 2), "GBps_aggregate": round(by / us / 1e3, 1), "gpus": world,
                                            "page_keys": 128}
            del kp, vp, ksp, vsp, ws
        except Exception as e:
            out["c5a_paged_batch8_131k"] = {"error": str(e)}
    # configuration 5b: batch 1 x 524288 keys, sharded by sequence chunks.  Two realisations of the exchange:
    #   "nccl": attention exports (o, m, l), NCCL all-gather of 16.6 KB per rank (torch.distributed), merge kernel;
    #   "peer": nomos_attn_seq_sharded -- one launch per rank: the attention kernel stores its rows into the peers'
    #           mailboxes over NVLink, waits for theirs and merges.
    # Both are checked against the oracle: every rank computes the exact fp64 partial of its own chunk on the host,
    # the partials are gathered on the host and merged by the oracle.
    if selected("c5b_seq_sharded_512k"):
        try:
            from nomos_nvfp4_b200.sharding import SeqShardGroup
            T5 = 524288 // world
            cache = make_layer_cache(torch, ops, dev, 1, NKV, T5, HD, 1005 + rank)
            qh = np.random.default_rng(5005).standard_normal((1, 1, NH, HD), dtype=np.float32)
            q = torch.from_numpy(qh).to(dev).to(torch.bfloat16)
            o = torch.zeros((NH, HD), dtype=torch.bfloat16, device=dev)
            part = torch.zeros((NH, HD + 2), dtype=torch.float32, device=dev)
            gathered = torch.zeros((world, NH, HD + 2), dtype=torch.float32, device=dev)
            k, v, ks, vs = cache
            common = dict(q=q, k_cache=k, v_cache=v, k_scales=ks, v_scales=vs, kv_fmt=ops.KV_I8, q_type=ops.BF16, nh=NH, nkv=NKV,
                          kvg=NH // NKV, l_hd=HD, cache_hd=HD, cache_cap=T5, klen=T5, softmax_scale=SOFTMAX_SCALE, flags=ops.SETTLED_CACHE)
            a = ops.make_args(partial_out=part, **common)
            wsb = ops.attn_workspace_bytes(a)
            ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
            a.workspace, a.ws_bytes = ws.data_ptr(), wsb

            def gather():
                if world > 1:
                    dist.all_gather_into_tensor(gathered, part)
                else:
                    gathered.copy_(part.unsqueeze(0))

            def fn():
                ops.attn_fused(stream, a)
                gather()
                ops.attn_merge_partials(stream, gathered, world, NH, HD, o, ops.BF16)

            n5 = max(10, iters // 4)
            us = time_call(torch, fn, n5)
            # the three phases bracketed by events (this serialises them; the sum can exceed the pipelined step time)
            ph = np.zeros(3)
            for _ in range(n5):
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
                ev[0].record(); ops.attn_fused(stream, a); ev[1].record(); gather(); ev[2].record()
                ops.attn_merge_partials(stream, gathered, world, NH, HD, o, ops.BF16); ev[3].record()
                torch.cuda.synchronize()
                ph += np.array([ev[i].elapsed_time(ev[i + 1]) for i in range(3)]) * 1000.0 / n5
            # peer-memory variant
            o2 = torch.zeros((NH, HD), dtype=torch.bfloat16, device=dev)
            a2 = ops.make_args(out=o2, out_type=ops.BF16, **common)
            a2.workspace, a2.ws_bytes = ws.data_ptr(), wsb

            def agb(b):
                if world == 1:
                    return [b]
                lst = [None] * world
                dist.all_gather_object(lst, b)
                return lst

            def worst(rc):
                """Largest status over the ranks: every rank takes the same branch after a failure on one of them."""
                if world > 1:
                    tt = torch.tensor([float(rc)], device=dev); dist.all_reduce(tt, op=dist.ReduceOp.MAX); rc = int(tt.item())
                return rc

            group, peer_rc, peer_err = None, 0, None
            try:
                group = SeqShardGroup(rank, world, NH, HD, agb, timeout_us=200000)
            except Exception as e:                          # e.g. no peer access between two of the GPUs
                peer_rc, peer_err = 1, repr(e)
            peer_rc = worst(peer_rc)
            if peer_rc == 0:
                group.decode(stream, a2)                    # one step first: a group that cannot exchange is not timed
                peer_rc = worst(group.status(stream))
            us_peer = time_call(torch, lambda: group.decode(stream, a2), n5) if peer_rc == 0 else float("inf")
            if peer_rc == 0:
                peer_rc = worst(group.status(stream))
            if world > 1:
                tt = torch.tensor([us, us_peer, *ph], device=dev); dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                us, us_peer, ph = float(tt[0]), float(tt[1]), tt[2:].cpu().numpy()
            # parity of both variants (fp32 outputs of one more step each) against the oracle
            o32 = torch.zeros((NH, HD), dtype=torch.float32, device=dev); o32p = torch.zeros_like(o32)
            ops.attn_fused(stream, a); gather(); ops.attn_merge_partials(stream, gathered, world, NH, HD, o32, ops.F32)
            a2.out, a2.out_type = o32p.data_ptr(), ops.F32
            if peer_rc == 0:
                group.decode(stream, a2)
                peer_rc = worst(group.status(stream))
            from oracle import oracle as orc
            orc.set_threads(max(1, (os.cpu_count() or 1) // world))
            _, pe = orc.attn_exact(orc.bf16_round(qh[0]), k[0].cpu().numpy(), v[0].cpu().numpy(), ks[0].cpu().numpy(), vs[0].cpu().numpy(),
                                   orc.KV_I8, NH, NKV, HD, HD, T5, query_base_pos=T5 - 1, softmax_scale=float(SOFTMAX_SCALE), want_partial=True)
            parts = [pe]
            if world > 1:
                parts = [None] * world
                dist.all_gather_object(parts, pe)
            want = orc.merge_partials(np.stack(parts), HD)
            by = algorithmic_bytes(NKV, NH // NKV, 524288, HD)
            out["c5b_seq_sharded_512k"] = {
                "us_per_layer": round(min(us, us_peer), 2), "GBps_aggregate": round(by / min(us, us_peer) / 1e3, 1), "gpus": world,
                "exchange": "peer stores, one launch per rank" if us_peer <= us else "NCCL all-gather + merge launch",
                "nccl_allgather_plus_merge": {"us_per_layer": round(us, 2), "phases_us": {"attention": round(float(ph[0]), 2),
                                              "all_gather": round(float(ph[1]), 2), "merge": round(float(ph[2]), 2)},
                                              "parity_rel_err": float(f"{rel_err(o32.cpu().numpy(), want):.3e}")},
                "peer_stores_one_launch": {"us_per_layer": round(us_peer, 2) if us_peer != float("inf") else None, "status": int(peer_rc),
                                           **({"error": peer_err} if peer_err else {}),
                                           "parity_rel_err": float(f"{rel_err(o32p.cpu().numpy(), want):.3e}")},
                "parity_bar": 2e-3}
            if group is not None:
                group.close()
            del cache, ws
        except Exception as e:
            out["c5b_seq_sharded_512k"] = {"error": repr(e)}
    return out


# --------------------------------------------------- reference arm / CPU baseline

class CpuReference:
    """The reference's own route for int8 row-scale KV, restated on the CPU (oracle/, kind "port"): window reader
    to a bf16 scratch (lib/kv_cache_quant.mojo:221-249), then bf16-operand attention with fp32 softmax
    (lib/attention_gpu.mojo:207-248).  It streams the SAME bytes as the GPU arm: the layers of host_layer_rows()
    with the GPU arm's seeds, quantised by the oracle (bit-identical to the library's quantize-on-write), and the
    GPU arm's queries.  The reference itself is Mojo GPU code and cannot run here."""

    def __init__(self, threads=None):
        from oracle import oracle as orc
        orc.build()
        self.orc = orc
        self.threads = int(threads or os.cpu_count() or 1)
        orc.set_threads(self.threads)
        self.layers = {}
        qrng = np.random.default_rng(2002)                      # rank 0's queries of the GPU arm
        self.q = [orc.bf16_round(qrng.standard_normal((1, 1, NH, HD), dtype=np.float32))[0, 0] * np.float32(SOFTMAX_SCALE)
                  for _ in range(NLAYERS)]
        self.kd = np.zeros((NKV, T, HD), np.uint16); self.vd = np.zeros_like(self.kd)
        self.scores = np.zeros((NH, T), np.float32); self.out = np.zeros((NH, HD), np.float32)

    def layer(self, i: int):
        if i not in self.layers:
            self.layers[i] = host_quantised_layer(layer_seed(i, 0, 0), NKV, T, HD)
        return self.layers[i]

    def step(self, i: int, heads: int) -> float:
        """One pass of the route over the first `heads` KV heads of layer i % NLAYERS; seconds."""
        orc, kvg = self.orc, NH // NKV
        k8, v8, ks, vs = self.layer(i % NLAYERS)
        q = np.ascontiguousarray(self.q[i % NLAYERS][:heads * kvg])
        t0 = time.perf_counter()
        orc.dequant_kv_i8_layer(k8, ks, self.kd, heads, T, HD, T, T, 0)
        orc.dequant_kv_i8_layer(v8, vs, self.vd, heads, T, HD, T, T, 0)
        orc.attn_decode_dense(q, self.kd, self.vd, self.scores, self.out, heads * kvg, heads, HD, HD, T, T, kvg, True)
        return time.perf_counter() - t0


def cpu_reference_leg(budget_s: float = 12.0) -> dict:
    """cpu_baseline of the GPU arm's line: the route timed on full layers (16 KV heads) for about budget_s seconds."""
    ref = CpuReference()
    ref.step(0, NKV)                                            # warm-up (also builds the layer)
    times, t_all, i = [], time.time(), 0
    while time.time() - t_all < budget_s and i < 400:
        times.append(ref.step(0, NKV)); i += 1
    best = float(np.mean(times))
    by = algorithmic_bytes(NKV, NH // NKV, T, HD)
    return {"value": round(by / best / 1e9, 3), "unit": UNIT, "cores": ref.threads, "kind": "port",
            "sample": f"{len(times)} passes over the full C2 layer 0 ({by / 1e6:.0f} MB each, the GPU arm's bytes): "
                      f"window reader -> bf16 scratch -> bf16 attention, OpenMP x{ref.threads}",
            "us_per_layer": round(best * 1e6, 1)}


def run_reference(args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    steps, warmup = max(1, args.steps), max(args.warmup, 3)
    ref = CpuReference()
    for i in range(NLAYERS):
        ref.layer(i)
    # size a step so that warm-up + steps stay near two minutes: a step covers `heads` of the 16 KV heads
    t_head = min(ref.step(0, 2), ref.step(1, 2)) / 2.0
    heads = int(max(1, min(NKV, 110.0 / (t_head * (steps + warmup)))))
    for i in range(warmup):
        ref.step(i, heads)
    t0 = time.perf_counter()
    for i in range(steps):
        ref.step(i, heads)
    dt = (time.perf_counter() - t0) / steps
    by = algorithmic_bytes(heads, NH // NKV, T, HD)
    val = by / dt / 1e9
    ms_layer = algorithmic_bytes(NKV, NH // NKV, T, HD) / (val * 1e9) * 1e3
    cb = {"value": round(val, 3), "unit": UNIT, "cores": ref.threads, "kind": "port",
          "sample": f"each step = {heads} of the 16 KV heads of one C2 layer ({by / 1e6:.0f} MB of the GPU arm's own bytes, "
                    f"{NLAYERS} layers cycled); window reader -> bf16 scratch -> bf16 attention, OpenMP x{ref.threads}; "
                    f"at N GPUs the job is N such sequences, the sample stays one"}
    return {
        "impl": "reference", "metric": METRIC, "value": round(val, 3), "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms_layer, 3), "us_per_layer": round(ms_layer * 1000, 1),
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 operands, fp32 accumulate (CPU restatement of the reference route)",
        "data": "synthetic", "config": workload_config(args.gpus),
        "note": "the reference is Mojo GPU code and cannot run here; this is its CPU restatement (oracle/); ms_per_step is "
                "the time of a full layer at the measured throughput",
        "cpu_baseline": cb,
        "e2e": {"value": round(val, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--quick", action="store_true", help="warm-up + timed steps only (for profiler captures)")
    ap.add_argument("--extras-only", action="store_true", help="run only the secondary configurations, --steps iterations each")
    ap.add_argument("--only", default=None, help="with --extras-only: comma-separated names of the cases to run")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle comparison of the timed outputs")
    args = ap.parse_args()
    if args.extras_only:
        import torch
        import torch.distributed as dist
        from nomos_nvfp4_b200 import ops
        torch.cuda.set_device(0)
        print(json.dumps({"extras": extras(torch, dist, ops, "cuda:0", 0, 1, iters=args.steps,
                                            only=set(args.only.split(",")) if args.only else None)}), flush=True)
        return
    res = run_reference(args) if args.impl == "reference" else run_ours(args)
    if res:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
