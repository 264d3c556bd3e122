#!/usr/bin/env python
"""Benchmark of the attention + KV-cache hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload ...]

Default workload ("c4"): long-context paged GQA decode with Llama-3.1-70B attention shapes
(64 q heads, 8 kv heads, head_dim 128, bf16, batch 32, every context 32768 tokens, block 64),
KV heads sharded across the N GPUs with no data-path collective.  One step = one decode pass of
the hot path over the batch, ONE launch: the split-KV decode kernel writes the new token's K/V
rows, streams the cache and merges its splits.  The headline value is decode-attention HBM GB/s:
algorithmic bytes of the batch divided by the step time (max over ranks).

One JSON line is printed by rank 0.  Besides the contract keys it carries
  roofline      the decode launch against the measured HBM peak,
  cpu_baseline  the CPU oracle port timed on a bounded sample on this machine's cores (N=1),
  e2e           the same metric through B200AttentionBackendImpl.forward with pinned HOST inputs
                copied in and the output copied back every step (the KV cache is the runner's
                resident state, as in the plugin),
  parity_check  the timed step's output rows of two users against the CPU oracle,
  sustained     the same step replayed for about two seconds (median and spread),
  prefill       the config-2 causal prefill (tcgen05 kernel) in TFLOP/s against the tensor peak,
  extra_workloads  configs 1 and 3 (decode rows), and for N > 1 the row-parallel linear,
  e2e_model     config 5: Llama-3.1-8B decode tokens/s through vLLM with this backend (TP = N);
                from N = 4 up also with the opt-in fused row-parallel linear
                (e2e_model_fused_linear).
`--impl reference` times the reference algorithm's CPU path (the oracle port; the Python
reference tree itself is not present on the GPU machine) on a bounded sample per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "tt-xla_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

# DRAM traffic of the split-KV decode kernel as one `ncu --set full -k regex:paged_decode_splitkv`
# capture of `bench.py --workload c4s` measured it: dram reads = 268.60 MB for 268.70 MB of
# algorithmic bytes, dram writes = 6.25 MB for 8.52 MB of fp32 split partials (the rest is still
# in L2 when it is merged).  Both parts grow in proportion to their own size, so a full launch
# is scaled from them.  These are constants of that capture, not a live measurement.
NCU_READ_PER_ALGORITHMIC_BYTE = 268.60 / 268.70
NCU_WRITE_PER_PARTIAL_BYTE = 6.25 / 8.52
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0

WORKLOADS = {
    # name: decode geometry
    "c4": dict(nq=64, nkv=8, hd=128, bs=64, users=32, ctx_lo=32768, ctx_hi=32768,
               desc="c4_long_context_decode_llama70b_B32_L32768"),
    "c3": dict(nq=32, nkv=8, hd=128, bs=64, users=64, ctx_lo=1024, ctx_hi=8192,
               desc="c3_decode_rows_llama8b_B64_L1024-8192"),
    "c1": dict(nq=32, nkv=8, hd=64, bs=32, users=8, ctx_lo=128, ctx_hi=1024,
               desc="c1_decode_llama1b_B8_L128-1024"),
    # config-4 geometry at a quarter of the context and a quarter of the batch: the case
    # profiler captures run on (268 MB of KV: larger than L2, small enough to replay)
    "c4s": dict(nq=64, nkv=8, hd=128, bs=64, users=8, ctx_lo=8192, ctx_hi=8192,
                desc="c4_small_decode_llama70b_B8_L8192"),
    "c4sf8": dict(nq=64, nkv=8, hd=128, bs=64, users=8, ctx_lo=8192, ctx_hi=8192,
                  kv_dtype="fp8_e4m3", desc="c4_small_decode_llama70b_B8_L8192_fp8kv"),
    # config 4 over an fp8 (e4m3) cache: half the bytes per token
    "c4f8": dict(nq=64, nkv=8, hd=128, bs=64, users=32, ctx_lo=32768, ctx_hi=32768,
                 kv_dtype="fp8_e4m3", desc="c4_long_context_decode_llama70b_B32_L32768_fp8kv"),
}


# ------------------------------------------------------------------------------ helpers
def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    source="measured")
    except Exception:
        return dict(hbm_gbs=FALLBACK_HBM_GBS, bf16_tflops=FALLBACK_BF16_TFLOPS, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons in the background during the timed region."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "power_w_max": max(power) if power else None,
                "reasons": sorted(reasons)}


def decode_algorithmic_bytes(ctx_lens: torch.Tensor, nq: int, nkv: int, hd: int, bs: int,
                             kv_elem_bytes: int = 2) -> int:
    """K and V rows of every context read once (the G query heads of a KV head share them),
    q read and o written, page-table entries and positions read."""
    users = ctx_lens.numel()
    kv = int(ctx_lens.sum()) * 2 * nkv * hd * kv_elem_bytes
    qo = 2 * users * nq * hd * 2
    meta = int(((ctx_lens + bs - 1) // bs).sum()) * 4 + 4 * users
    return kv + qo + meta


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier(world: int):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ------------------------------------------------------------------------------ workloads
class StagedInputs:
    """One pinned host buffer and one device buffer holding a step's inputs back to back (256-byte
    aligned segments), so that a step's host-to-device transfer is a single copy."""

    def __init__(self, tensors: dict, device):
        self.offsets, total = {}, 0
        for name, t in tensors.items():
            self.offsets[name] = total
            total += (t.numel() * t.element_size() + 255) // 256 * 256
        self.host = torch.empty(total, dtype=torch.uint8).pin_memory()
        self.dev = torch.empty(total, dtype=torch.uint8, device=device)
        self.nbytes = total
        self.h, self.d = {}, {}
        for name, t in tensors.items():
            o, n = self.offsets[name], t.numel() * t.element_size()
            self.h[name] = self.host[o:o + n].view(t.dtype).view(t.shape)
            self.d[name] = self.dev[o:o + n].view(t.dtype).view(t.shape)
            self.h[name].copy_(t)

    def upload(self):
        self.dev.copy_(self.host, non_blocking=True)


def make_decode_workload(wl: dict, rank: int, world: int, device):
    """Per-rank tensors of the decode workload: this rank's KV heads of every block (allocated
    the way the plugin's runner allocates them, then filled with N(0,1)), its q heads, and a
    replica of the int32 metadata."""
    from b200attn import sharding

    nq, nkv, hd, bs, users = wl["nq"], wl["nkv"], wl["hd"], wl["bs"], wl["users"]
    if nkv % world != 0:
        raise SystemExit(f"{nkv} kv heads do not shard over {world} GPUs")
    g = torch.Generator().manual_seed(4)
    ctx = torch.randint(wl["ctx_lo"], wl["ctx_hi"] + 1, (users,), generator=g)
    nblk = (wl["ctx_hi"] + bs - 1) // bs
    nb = users * nblk
    page_table = torch.randperm(nb, generator=g).reshape(users, nblk).to(torch.int32)
    nkv_l, nq_l = nkv // world, nq // world
    kv_dtype = torch.float8_e4m3fn if wl.get("kv_dtype") == "fp8_e4m3" else torch.bfloat16
    k_cache, v_cache = sharding.allocate_kv_caches(["layer"], nb, nkv, bs, hd, dtype=kv_dtype,
                                                   device=device, tp_size=world)["layer"]
    fill_cache_randn(k_cache, 100 + rank)
    fill_cache_randn(v_cache, 200 + rank)
    gq = torch.Generator().manual_seed(300 + rank)
    inputs = dict(
        q=torch.randn(users, nq_l * hd, generator=gq).to(torch.bfloat16),
        k=torch.randn(users, nkv_l * hd, generator=gq).to(torch.bfloat16),
        v=torch.randn(users, nkv_l * hd, generator=gq).to(torch.bfloat16),
        cache_position=(ctx - 1).to(torch.int32),
        page_table=page_table,
    )
    return dict(nq=nq_l, nkv=nkv_l, hd=hd, bs=bs, users=users, ctx=ctx, nb=nb,
                k_cache=k_cache, v_cache=v_cache, inputs=inputs, max_ctx=int(ctx.max()))


def fill_cache_randn(cache: torch.Tensor, seed: int) -> None:
    """N(0,1) into an allocated cache, block range by block range so the fp32 temporaries stay
    small."""
    nb, nkv, bs, hd = cache.shape
    g = torch.Generator(device=cache.device).manual_seed(seed)
    step = max(1, (256 << 20) // (nkv * bs * hd * 4))
    for b0 in range(0, nb, step):
        b1 = min(nb, b0 + step)
        cache[b0:b1] = torch.randn((b1 - b0, nkv, bs, hd), generator=g, device=cache.device,
                                   dtype=torch.float32).to(cache.dtype)


def oracle_check(w, out: torch.Tensor, users_to_check) -> dict:
    """Compares the timed step's output rows of a few users with the CPU oracle (fp32 arithmetic
    on the same cache contents, new token included), this rank's heads."""
    from oracle import restate

    nq, nkv, hd, bs = w["nq"], w["nkv"], w["hd"], w["bs"]
    G = nq // nkv
    scale = hd ** -0.5
    pt = w["inputs"]["page_table"]
    worst, total, count = 0.0, 0.0, 0
    for u in users_to_check:
        L = int(w["ctx"][u])
        pages = pt[u, : (L + bs - 1) // bs].long()
        kc = w["k_cache"][pages.to(w["k_cache"].device)].float().cpu()      # [pages, nkv, bs, hd]
        vc = w["v_cache"][pages.to(w["v_cache"].device)].float().cpu()
        local_pt = torch.arange(pages.numel(), dtype=torch.int32)[None]
        q = w["inputs"]["q"][u].view(1, 1, nq, hd).float()
        pos = torch.tensor([L - 1], dtype=torch.int32)
        got = out[u].float().cpu().view(nq, hd)
        for h in range(nkv):
            want = restate.paged_sdpa_decode(q[:, :, h * G:(h + 1) * G], kc[:, h:h + 1],
                                             vc[:, h:h + 1], local_pt, pos, scale)[0, 0]
            d = (got[h * G:(h + 1) * G] - want).abs()
            worst = max(worst, float(d.max()))
            total += float(d.sum())
            count += d.numel()
    return {"users": list(users_to_check), "max_abs": worst, "mean_abs": total / max(count, 1)}


def run_decode_bench(args, wl, rank, world, device, light: bool = False):
    """Times the decode step of workload `wl`.  `light`: device-timed graph replays only (the
    extra workloads reported beside the headline one)."""
    from b200attn import B200AttentionBackendImpl, B200Metadata, ops

    w = make_decode_workload(wl, rank, world, device)
    users, nq, nkv, hd, bs = w["users"], w["nq"], w["nkv"], w["hd"], w["bs"]
    staged = StagedInputs(w["inputs"], device)
    staged.upload()
    dev = staged.d
    out = torch.empty(users, nq * hd, dtype=torch.bfloat16, device=device)
    q3 = dev["q"].view(users, nq, hd)
    k3 = dev["k"].view(users, nkv, hd)
    v3 = dev["v"].view(users, nkv, hd)
    out3 = out.view(users, nq, hd)
    scale = hd ** -0.5
    splits = ops.decode_auto_splits(users, nkv, hd, w["max_ctx"])

    def step():
        ops.paged_decode(q3, w["k_cache"], w["v_cache"], dev["page_table"], dev["cache_position"],
                         scale=scale, out=out3, num_splits=splits, max_context_len=w["max_ctx"],
                         new_key=k3, new_value=v3)

    ops.read_error_word()
    for _ in range(args.warmup):
        step()
    # ---- timed region: K steps, device events, max over ranks; per-step decode-call events too
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(args.steps)]
    sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 and not light else None
    barrier(world)
    if sampler:
        sampler.start()
        time.sleep(0.3)
    barrier(world)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(args.steps):
        ev[i][0].record()
        step()
        ev[i][1].record()
    t1.record()
    barrier(world)
    eager_ms = max_over_ranks(t0.elapsed_time(t1), world, device)
    # The same K steps replayed as a CUDA graph of one step: how a serving loop runs a decode
    # step (vLLM replays decode as full CUDA graphs); removes the host launch gaps that matter
    # once the per-GPU step is down to ~0.1 ms.
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()                                  # workspace of this stream exists before capture
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph, stream=side):
        step()
    for _ in range(3):
        graph.replay()
    barrier(world)
    g0 = torch.cuda.Event(enable_timing=True)
    g1 = torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(args.steps):
        graph.replay()
    g1.record()
    barrier(world)
    total_ms = max_over_ranks(g0.elapsed_time(g1), world, device)
    decode_ms = statistics.mean(a.elapsed_time(b) for a, b in ev)
    decode_ms = max_over_ranks(decode_ms, world, device)
    eb = w["k_cache"].element_size()
    full_bytes = decode_algorithmic_bytes(w["ctx"], wl["nq"], wl["nkv"], hd, bs, eb)
    rank_bytes = decode_algorithmic_bytes(w["ctx"], nq, nkv, hd, bs, eb)
    ms_per_step = total_ms / args.steps
    res = dict(w=w, full_bytes=full_bytes, rank_bytes=rank_bytes, ms_per_step=ms_per_step,
               decode_ms=decode_ms, eager_ms_per_step=eager_ms / args.steps, splits=splits,
               launches=args.steps, out=out,
               partial_bytes=ops.decode_workspace_bytes(users, nq, hd, splits))
    if light:
        err = ops.read_error_word()
        if err:
            raise SystemExit(f"a kernel reported device error {err}")
        return res

    # ---- sustained: rounds of K replays for about two seconds, each round timed on its own
    rounds, spent = [], 0.0
    while spent < args.sustain_s * 1e3 and len(rounds) < 2000:
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            graph.replay()
        b.record()
        b.synchronize()
        rounds.append(a.elapsed_time(b) / args.steps)
        spent += rounds[-1] * args.steps
    barrier(world)
    clocks = sampler.stop() if sampler else None
    if rounds:
        srt = sorted(rounds)
        med = max_over_ranks(statistics.median(rounds), world, device)
        res["sustained"] = {
            "seconds": round(spent / 1e3, 2), "rounds": len(rounds),
            "ms_per_step_median": round(med, 4),
            "ms_per_step_p05": round(srt[len(srt) // 20], 4),
            "ms_per_step_p95": round(srt[min(len(srt) - 1, len(srt) * 19 // 20)], 4),
            "value_median": round(full_bytes / (med * 1e-3) / 1e9, 1), "unit": "GB/s"}
    err = ops.read_error_word()
    if err:
        raise SystemExit(f"a kernel reported device error {err}")

    # ---- parity of what was timed: a few users' rows against the CPU oracle
    check = oracle_check(w, out, sorted({0, users - 1}))
    check["max_abs"] = max_over_ranks(check["max_abs"], world, device)
    check["mean_abs"] = max_over_ranks(check["mean_abs"], world, device)
    check["tolerance"] = {"max_abs": 2e-2, "mean_abs": 2e-3}
    check["ok"] = check["max_abs"] <= 2e-2 and check["mean_abs"] <= 2e-3
    res["parity_check"] = check

    # ---- e2e: through the backend's forward; the step's inputs go host -> device in ONE copy of
    # a pinned staging buffer, the output comes back in one copy, the host waits for it
    impl = B200AttentionBackendImpl(nq, hd, scale, nkv, None, None,
                                    "fp8_e4m3" if wl.get("kv_dtype") == "fp8_e4m3" else "auto")
    kv = [w["k_cache"], w["v_cache"]]
    md = B200Metadata(cache_position=dev["cache_position"], page_table=dev["page_table"],
                      num_users=users,
                      batch_idx=torch.arange(users, dtype=torch.int32, device=device),
                      max_seq_len=w["max_ctx"])
    h_out = torch.empty(users, nq * hd, dtype=torch.bfloat16).pin_memory()
    h2d, d2h = staged.nbytes, h_out.numel() * h_out.element_size()

    def e2e_body():
        staged.upload()
        impl.forward(None, dev["q"], dev["k"], dev["v"], kv, md, output=out)
        h_out.copy_(out, non_blocking=True)

    def timed_e2e(run_one):
        for _ in range(max(3, args.warmup)):
            run_one()
        barrier(world)
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            run_one()
        e1.record()
        barrier(world)
        return max_over_ranks(e0.elapsed_time(e1), world, device) / args.steps

    def eager_one():
        e2e_body()
        torch.cuda.current_stream().synchronize()

    e2e_eager_ms = timed_e2e(eager_one)
    # The same step (copy in, forward, copy out) captured once and replayed, the way a serving
    # engine runs a decode step; the host still waits for every step's output.
    e2e_graph = torch.cuda.CUDAGraph()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        e2e_body()
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(e2e_graph, stream=side):
        e2e_body()

    def graph_one():
        e2e_graph.replay()
        torch.cuda.current_stream().synchronize()

    e2e_ms = timed_e2e(graph_one)
    e2e_check = (h_out.float() - out.float().cpu()).abs().max().item()
    res.update(e2e_ms=e2e_ms, e2e_eager_ms=e2e_eager_ms, h2d=h2d, d2h=d2h, clocks=clocks,
               e2e_readback_matches=e2e_check == 0.0)
    return res


def run_prefill_bench(args, rank, world, device, peaks):
    """Config 2: 4 x 2048 tokens, nq 32 / nkv 8 / hd 128, block 64, heads sharded over the ranks.
    One step = paged_fill_cache + causal prefill attention on the fresh K/V."""
    from b200attn import ops

    users, T, nq, nkv, hd, bs = 4, 2048, 32 // world, 8 // world, 128, 64
    if nkv == 0:
        return None
    g = torch.Generator(device=device).manual_seed(7 + rank)
    q = torch.randn(users * T, nq, hd, generator=g, device=device).bfloat16()
    k = torch.randn(users * T, nkv, hd, generator=g, device=device).bfloat16()
    v = torch.randn(users * T, nkv, hd, generator=g, device=device).bfloat16()
    nblk = T // bs
    nb = users * nblk + 1
    pt = (torch.randperm(nb - 1)[: users * nblk] + 1).reshape(users, nblk).int().to(device)
    kc = torch.zeros(nb, nkv, bs, hd, dtype=torch.bfloat16, device=device)
    vc = torch.zeros_like(kc)
    out = torch.empty_like(q)
    cu_host = torch.arange(users + 1, dtype=torch.int32) * T
    cu_dev = cu_host.to(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    k4, v4 = k.view(users, T, nkv, hd), v.view(users, T, nkv, hd)
    steps = max(3, min(args.steps, 20))
    times = []
    for i in range(3 + steps):
        flush.zero_()  # 256 MiB write: evicts the 126 MB L2 between iterations
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        c = torch.cuda.Event(enable_timing=True)
        a.record()
        ops.paged_fill_cache(kc, vc, k4, v4, pt)
        b.record()
        ops.prefill(q, k, v, cu_host, scale=hd ** -0.5, out=out, cu_q=cu_dev)
        c.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append((a.elapsed_time(b), b.elapsed_time(c)))
    fill_ms = max_over_ranks(statistics.mean(t[0] for t in times), world, device)
    attn_ms = max_over_ranks(statistics.mean(t[1] for t in times), world, device)
    flops_full = 4 * hd * 32 * users * (T * (T + 1) // 2)
    tflops = flops_full / (attn_ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops"] * world
    return {"workload": "c2_causal_prefill_llama8b_4x2048", "tflops": round(tflops, 1),
            "attn_ms": round(attn_ms, 4), "fill_cache_ms": round(fill_ms, 4),
            "flops": flops_full, "l2": "flushed between iterations",
            "roofline": {"bound": "tensor", "achieved": round(tflops, 1), "peak": peak,
                         "unit": "TFLOP/s", "frac": round(tflops / peak, 4),
                         "peak_source": peaks["source"]}}


def run_chunk_bench(args, rank, world, device, peaks):
    """The prefill half of config 3: 2 chunks of 512 tokens appended to contexts of 4096 already in
    the paged cache (nq 32 / nkv 8 / hd 128, block 64), heads sharded over the ranks.  One step =
    paged_fill_cache of the chunk + chunked prefill attention over prefix + chunk."""
    from b200attn import ops

    users, T, start, nq, nkv, hd, bs = 2, 512, 4096, 32 // world, 8 // world, 128, 64
    if nkv == 0:
        return None
    g = torch.Generator(device=device).manual_seed(11 + rank)
    q = torch.randn(users * T, nq, hd, generator=g, device=device).bfloat16()
    k = torch.randn(users, T, nkv, hd, generator=g, device=device).bfloat16()
    v = torch.randn(users, T, nkv, hd, generator=g, device=device).bfloat16()
    nblk = (start + T) // bs
    nb = users * nblk + 1
    pt = (torch.randperm(nb - 1)[: users * nblk] + 1).reshape(users, nblk).int().to(device)
    fpt = torch.roll(pt, -(start // bs), dims=1).contiguous()
    kc = torch.randn(nb, nkv, bs, hd, generator=g, device=device).bfloat16()
    vc = torch.randn(nb, nkv, bs, hd, generator=g, device=device).bfloat16()
    out = torch.empty_like(q)
    cu_host = torch.arange(users + 1, dtype=torch.int32) * T
    cu_dev = cu_host.to(device)
    q_start = torch.full((users,), start, dtype=torch.int32, device=device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    times = []
    for i in range(3 + 10):
        flush.zero_()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        ops.paged_fill_cache(kc, vc, k, v, fpt)
        ops.prefill(q, kc, vc, cu_host, scale=hd ** -0.5, page_table=pt, q_start=q_start,
                    out=out, cu_q=cu_dev)
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(a.elapsed_time(b))
    ms = max_over_ranks(statistics.mean(times), world, device)
    flops = 4 * hd * 32 * users * (T * start + T * (T + 1) // 2)
    tflops = flops / (ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops"] * world
    return {"workload": "c3_chunks_2x512_on_prefix_4096", "tflops": round(tflops, 1),
            "ms": round(ms, 4), "flops": flops, "l2": "flushed between iterations",
            "note": "2 sequences x 32 heads x 2 row blocks = 128 work items for 148 SMs",
            "roofline": {"bound": "tensor", "achieved": round(tflops, 1), "peak": peak,
                         "unit": "TFLOP/s", "frac": round(tflops / peak, 4),
                         "peak_source": peaks["source"]}}


# ------------------------------------------------------------------------------ config 5
LLAMA31_8B = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=4096,
                  intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                  num_key_value_heads=8, head_dim=128, vocab_size=128256, rope_theta=500000.0,
                  max_position_embeddings=8192, rms_norm_eps=1e-5, torch_dtype="bfloat16",
                  tie_word_embeddings=False, hidden_act="silu", bos_token_id=1, eos_token_id=2)


def measure_rowlinear(args, rank, world, device, steps=None):
    """Row-parallel linear + all-reduce of the end-to-end model's decode step (config 5: 64 token
    rows, hidden 4096, o_proj K = 4096 / TP and down_proj K = 14336 / TP): the fused launch of
    this repository against torch's GEMM followed by an NCCL all-reduce, both walking a set of 32
    different weight matrices (one per layer, larger than L2 together) as the model does.  Device
    time by CUDA events, max over ranks.  Also checks the fused result: error against an fp32
    all-reduce of fp32 partial products, and that every rank holds the same bits."""
    from b200attn import ops, tp_linear

    steps = steps or args.steps
    comm = tp_linear.RowLinearComm(dist.group.WORLD, max_n=4096, max_tokens=128) if world > 1 else None
    tokens, hidden, layers = 64, 4096, 32
    results = {}
    for name, k_full in (("o_proj", 4096), ("down_proj", 14336)):
        kl = k_full // world
        g = torch.Generator(device=device).manual_seed(7 + rank)
        ws = [(torch.randn(hidden, kl, generator=g, device=device) * 0.02).to(torch.bfloat16)
              for _ in range(layers)]
        x = torch.randn(tokens, kl, generator=g, device=device).to(torch.bfloat16)
        out = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=device)

        def fused(mode=0):
            for w in ws:
                tp_linear.rowlinear_allreduce(x, w, comm, out=out, reduce_mode=mode)

        def stock():
            for w in ws:
                torch.matmul(x, w.t(), out=out)
                if world > 1:
                    dist.all_reduce(out)

        def timed(fn):
            # one pass over the 32 layers captured as a CUDA graph (how the serving engine runs
            # its decode steps), so that device time is measured and not Python launch time
            fn()
            barrier(world)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
            for _ in range(args.warmup):
                graph.replay()
            barrier(world)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            return max_over_ranks(e0.elapsed_time(e1) * 1e3 / (steps * layers), world, device)

        us_stock = timed(stock)
        us_fused = timed(fused)
        by_mode = {}
        if world > 2:       # both exchange schemes, for the record (the default picks two shots)
            by_mode = {"one_shot_us": round(timed(lambda: fused(1)), 2),
                       "two_shot_us": round(timed(lambda: fused(2)), 2)}
        # correctness of what was timed: last layer's result against fp32 arithmetic
        tp_linear.rowlinear_allreduce(x, ws[-1], comm, out=out)
        ref = x.float() @ ws[-1].float().t()
        if world > 1:
            dist.all_reduce(ref)
        err = max_over_ranks(float((out.float() - ref).abs().max()), world, device)
        digest = out.view(torch.int16).to(torch.int64).sum().reshape(1)
        same = True
        if world > 1:
            digests = [torch.empty_like(digest) for _ in range(world)]
            dist.all_gather(digests, digest)
            same = all(int(d) == int(digests[0]) for d in digests)
        wbytes = hidden * kl * 2
        results[name] = {"k_local": kl, "fused_us": round(us_fused, 2), "stock_us": round(us_stock, 2),
                         "weight_gbs_fused": round(wbytes / us_fused / 1e3, 1),
                         "weight_gbs_stock": round(wbytes / us_stock / 1e3, 1),
                         "max_abs_err_vs_fp32": round(err, 5), "all_ranks_identical": same,
                         **by_mode}
    word = ops.read_error_word()
    if comm is not None:
        dist.barrier()
        comm.close()
    results["error_word"] = word
    results["stock"] = "torch.matmul + NCCL all-reduce"
    results["form"] = "64 token rows, N 4096, 32 distinct weights per pass, CUDA-graph replay"
    return results


def run_rowlinear_bench(args):
    rank, world, local = dist_setup(args.gpus)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    peaks = load_peaks()
    results = measure_rowlinear(args, rank, world, device)
    if rank == 0:
        o = results["o_proj"]
        print(json.dumps({
            "metric": "rowlinear_allreduce_us", "value": o["fused_us"], "unit": "us", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(o["fused_us"] * 32e-3, 4),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "c5_rowparallel_linear_allreduce_B64_hidden4096",
                       "parallelism": f"tp{world}", "step": "32 layers back to back, replayed as one CUDA graph",
                       "l2": "32 distinct weight matrices per pass (larger than L2 together)",
                       "stock": "torch.matmul + NCCL all-reduce"},
            "layers": results, "error_word": results["error_word"],
            "roofline": {"bound": "hbm", "achieved": o["weight_gbs_fused"], "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": round(o["weight_gbs_fused"] / peaks["hbm_gbs"], 4),
                         "traffic": None, "peak_source": peaks["source"],
                         "note": "weight bytes of one o_proj launch / its device time, all-reduce "
                                 "included in the time"},
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_e2e_model_subprocess(args, rank: int, world: int, timeout_s: int = 600,
                             port_offset: int = 23):
    """Config 5 (end-to-end Llama-3.1-8B decode through vLLM, `--workload c5`) as a child process
    of every rank, so that the engine gets a fresh CUDA context and its own process group.
    Returns rank 0's result line as a dict (None on the other ranks)."""
    env = dict(os.environ)
    if world > 1:
        # a rendezvous of its own: the parent's store keeps serving the parent's group
        env["MASTER_PORT"] = str(int(env.get("MASTER_PORT", "29500")) + port_offset)
        for k in ("TORCHELASTIC_USE_AGENT_STORE", "TORCHELASTIC_RUN_ID", "TORCHELASTIC_RESTART_COUNT",
                  "TORCHELASTIC_MAX_RESTARTS", "TORCHELASTIC_ERROR_FILE"):
            env.pop(k, None)
    cmd = [sys.executable, os.path.abspath(__file__), "--workload", "c5", "--gpus", str(world),
           "--steps", "1"]
    if args.fused_linear:
        cmd.append("--fused-linear")
    try:
        proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout_s)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"config 5 did not finish within {timeout_s} s"} if rank == 0 else None
    if rank != 0:
        return None
    for ln in reversed(proc.stdout.splitlines()):
        if ln.startswith("{") and '"e2e_decode_tokens_per_s"' in ln:
            d = json.loads(ln)
            return {"metric": d["metric"], "value": d["value"], "unit": d["unit"],
                    "ms_per_step": d["ms_per_step"], "ttft_s": d["ttft_s"],
                    "generate_s": d["generate_s"], "tokens": d["tokens"],
                    "error_word": d["error_word"], "config": d["config"],
                    "roofline": d["roofline"]}
    tail = (proc.stderr or proc.stdout)[-400:].replace("\n", " | ")
    return {"unavailable": f"config 5 child exited {proc.returncode}: {tail}"}


def run_e2e_llama(args):
    """Config 5: end-to-end decode of a random-init Llama-3.1-8B through vLLM with this
    repository's backend registered as the CUSTOM attention backend (the way the reference
    plugin registers its own).  Batch 64, prompts of 1024 uniform-random token ids, 256 output
    tokens each, greedy, no EOS.  Tensor parallel = number of ranks (torchrun); vLLM's own NCCL
    all-reduce follows o_proj and down_proj.  Decode steps replay as CUDA graphs."""
    import tempfile

    pkg = os.path.join(ROOT, "tt-xla_b200")
    os.environ["PYTHONPATH"] = pkg + os.pathsep + os.environ.get("PYTHONPATH", "")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1:
        os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"
    # explicit either way, so that the line says what ran (the plugin's own default is "auto")
    os.environ["B200ATTN_FUSED_ROW_PARALLEL"] = "1" if args.fused_linear else "0"
    from vllm import LLM, SamplingParams

    cfg_dir = tempfile.mkdtemp(prefix="llama31_8b_cfg_")
    with open(os.path.join(cfg_dir, "config.json"), "w") as f:
        json.dump(LLAMA31_8B, f)
    batch, prompt_len, gen_len = 64, 1024, 256
    kw = dict(model=cfg_dir, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16",
              block_size=64, max_model_len=2048, max_num_seqs=batch, max_num_batched_tokens=8192,
              gpu_memory_utilization=0.85, seed=0, enable_prefix_caching=False,
              tensor_parallel_size=world, enforce_eager=False,
              compilation_config={"mode": 0, "cudagraph_mode": "FULL_DECODE_ONLY"})
    if args.attn == "b200":
        kw["attention_backend"] = "CUSTOM"
    if world > 1:
        kw["distributed_executor_backend"] = "external_launcher"
    llm = LLM(**kw)
    g = torch.Generator().manual_seed(0)
    prompts = [dict(prompt_token_ids=torch.randint(0, LLAMA31_8B["vocab_size"], (prompt_len,),
                                                   generator=g).tolist()) for _ in range(batch)]

    def timed(max_tokens):
        sp = SamplingParams(max_tokens=max_tokens, ignore_eos=True, temperature=0.0,
                            detokenize=False)
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp, use_tqdm=False)
        dt = time.perf_counter() - t0
        return dt, sum(len(o.outputs[0].token_ids) for o in outs)

    timed(8)                                   # warm-up: graphs captured, allocator settled
    reps = max(1, min(args.steps, 3))
    t_first = min(timed(1)[0] for _ in range(reps))        # prefill + first token
    full = [timed(gen_len) for _ in range(reps)]
    t_full = min(f[0] for f in full)
    n_tok = full[0][1]
    decode_s = t_full - t_first
    decode_tok = batch * (gen_len - 1)
    tok_s = decode_tok / decode_s
    err_word = None
    if world > 1:          # the engine runs in this process: its kernels' diagnostics word is ours
        from b200attn import ops
        err_word = ops.read_error_word()
    # stop the engine first so that its shutdown messages do not follow the result line
    try:
        llm.llm_engine.engine_core.shutdown()
    except Exception:
        pass
    del llm
    time.sleep(1.0)
    if rank == 0:
        step_ms = decode_s / (gen_len - 1) * 1e3
        weights = 2 * (LLAMA31_8B["vocab_size"] * 4096 * 2 + 32 * (4096 * 6144 + 4096 * 4096 +
                                                                    3 * 4096 * 14336))
        kv_per_step = batch * (prompt_len + gen_len / 2) * 32 * 2 * 8 * 128 * 2
        peaks = load_peaks()
        gbs = (weights + kv_per_step) / world / (step_ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "e2e_decode_tokens_per_s", "value": round(tok_s, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": reps, "warmup": 1, "ms_per_step": round(step_ms, 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "c5_llama31_8b_e2e_decode_B64_P1024_G256",
                       "parallelism": f"tp{world}", "attention_backend": args.attn,
                       "row_parallel_linear": "fused GEMM + all-reduce" if args.fused_linear
                       else "vLLM GEMM + all-reduce",
                       "weights": "random init (vLLM dummy loader)",
                       "timing": "wall clock around LLM.generate; decode = (256-token run) - "
                                 "(1-token run); decode steps are CUDA-graph replays"},
            "ttft_s": round(t_first, 4), "generate_s": round(t_full, 4), "tokens": n_tok,
            "error_word": err_word,
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4),
                         "traffic": None, "peak_source": peaks["source"],
                         "note": "per-GPU bytes of one decode step = bf16 weights / TP + mean "
                                 "KV of the batch / TP"},
        }), flush=True)


# ------------------------------------------------------------------------------ CPU side
def cpu_decode_sample(wl: dict, n_users: int, seed: int = 0):
    """A bounded sample of the decode workload for the CPU oracle: n_users users of the batch,
    all heads, native bf16 (the dtype the reference's CPU branch would compute in)."""
    nq, nkv, hd, bs = wl["nq"], wl["nkv"], wl["hd"], wl["bs"]
    g = torch.Generator().manual_seed(1000 + seed)
    ctx = torch.randint(wl["ctx_lo"], wl["ctx_hi"] + 1, (n_users,), generator=g)
    nblk = (wl["ctx_hi"] + bs - 1) // bs
    nb = n_users * nblk
    pt = torch.randperm(nb, generator=g).reshape(n_users, nblk).to(torch.int32)
    kc = torch.randn(nb, nkv, bs, hd, generator=g).to(torch.bfloat16)
    vc = torch.randn(nb, nkv, bs, hd, generator=g).to(torch.bfloat16)
    q = torch.randn(1, n_users, nq, hd, generator=g).to(torch.bfloat16)
    k = torch.randn(1, n_users, nkv, hd, generator=g).to(torch.bfloat16)
    v = torch.randn(1, n_users, nkv, hd, generator=g).to(torch.bfloat16)
    return dict(ctx=ctx, pt=pt, kc=kc, vc=vc, q=q, k=k, v=v, pos=(ctx - 1).to(torch.int32))


def cpu_cache_write(s):
    """The reference's decode-step cache write on CPU: `paged_update_cache` for K and for V.  The
    op is functional, so each call clones the whole pool (custom_ops.py:982); that clone is
    part of what the reference does and dominates this timing."""
    from oracle import restate

    kc = restate.paged_update_cache(s["kc"], s["k"], s["pos"], s["pt"])
    vc = restate.paged_update_cache(s["vc"], s["v"], s["pos"], s["pt"])
    return kc, vc


def cpu_decode_attention(s, kc, vc, hd: int):
    """The reference's paged decode attention on CPU over an already written cache."""
    from oracle import restate

    return restate.paged_sdpa_decode(s["q"], kc, vc, s["pt"], s["pos"], hd ** -0.5)


def time_cpu(fn, budget_s: float, max_reps: int = 50):
    reps, spent = 0, 0.0
    while reps < 1 or (spent < budget_s and reps < max_reps):
        t0 = time.perf_counter()
        fn()
        spent += time.perf_counter() - t0
        reps += 1
    return spent / reps, reps, spent


def run_cpu_baseline(wl: dict, budget_s: float = 12.0, max_users: int = 16):
    """Times the oracle port on a bounded sample: up to `max_users` users of the batch.  The
    decode attention and the cache write are timed apart: `value` is the attention alone (the
    metric is attention bytes per second); the write, whose cost on CPU is the functional clone
    of the whole pool, is reported beside it."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    s = cpu_decode_sample(wl, 1)
    kc, vc = cpu_cache_write(s)
    t0 = time.perf_counter()
    cpu_decode_attention(s, kc, vc, wl["hd"])
    t1 = time.perf_counter() - t0
    users = int(max(1, min(max_users, wl["users"], 0.75 * budget_s / max(t1, 1e-3))))
    if users > 1:
        s = cpu_decode_sample(wl, users)
        kc, vc = cpu_cache_write(s)
    attn_s, reps, spent = time_cpu(lambda: cpu_decode_attention(s, kc, vc, wl["hd"]),
                                   0.75 * budget_s)
    write_s, wreps, wspent = time_cpu(lambda: cpu_cache_write(s), 0.25 * budget_s, 10)
    nbytes = decode_algorithmic_bytes(s["ctx"], wl["nq"], wl["nkv"], wl["hd"], wl["bs"])
    return {"value": round(nbytes / attn_s / 1e9, 4), "unit": "GB/s", "cores": cores,
            "kind": "port",
            "attention_ms": round(attn_s * 1e3, 2), "cache_write_ms": round(write_s * 1e3, 2),
            "value_with_cache_write": round(nbytes / (attn_s + write_s) / 1e9, 4),
            "sample": f"{users} of {wl['users']} users of the batch, all heads, native bf16; decode "
                      f"attention alone: {reps} repetitions, {spent:.1f} s; cache write (two "
                      f"functional clones of the sample's pool): {wreps} repetitions, {wspent:.1f} s"}


def run_reference_arm(args, wl):
    """The reference algorithm's CPU path (oracle port) on this machine's cores: every step is
    the paged decode attention of one user of the batch (the cache write is timed apart and
    reported beside it: on CPU it is a functional clone of the pool)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    s = cpu_decode_sample(wl, 1)
    nbytes = decode_algorithmic_bytes(s["ctx"], wl["nq"], wl["nkv"], wl["hd"], wl["bs"])
    kc, vc = cpu_cache_write(s)
    for _ in range(args.warmup):
        cpu_decode_attention(s, kc, vc, wl["hd"])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_decode_attention(s, kc, vc, wl["hd"])
    dt = (time.perf_counter() - t0) / args.steps
    write_s, _, _ = time_cpu(lambda: cpu_cache_write(s), 2.0, 5)
    val = round(nbytes / dt / 1e9, 4)
    sample = (f"1 of {wl['users']} users per step, all heads, native bf16, decode attention "
              f"{dt:.2f} s per step; cache write apart: {write_s:.2f} s")
    print(json.dumps({
        "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(wl, args.gpus, parallelism="cpu host cores"),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port",
                         "cache_write_ms": round(write_s * 1e3, 2), "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def workload_config(wl: dict, world: int, parallelism: str) -> dict:
    """The `config` object both arms print: the workload and its geometry."""
    return {"workload": wl["desc"], "parallelism": parallelism, "q_heads": wl["nq"],
            "kv_heads": wl["nkv"], "head_dim": wl["hd"], "block_size": wl["bs"],
            "batch": wl["users"], "kv_cache_dtype": wl.get("kv_dtype", "bf16"),
            "context": [wl["ctx_lo"], wl["ctx_hi"]]}


# ------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS) + ["c5", "rowlinear"])
    ap.add_argument("--attn", default="b200", choices=["b200", "stock"],
                    help="c5 only: this repository's backend, or vLLM's stock one for comparison")
    ap.add_argument("--fused-linear", action="store_true",
                    help="c5: o_proj / down_proj through the fused GEMM + all-reduce launch")
    ap.add_argument("--sustain-s", type=float, default=2.0,
                    help="seconds of back-to-back graph replays reported beside the K-step number")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the extra workloads (configs 1 and 3, the row-parallel linear)")
    ap.add_argument("--no-e2e-model", action="store_true",
                    help="skip config 5 (end-to-end Llama-3.1-8B through vLLM, a child process)")
    ap.add_argument("--only", default="all", choices=["all", "prefill"],
                    help="prefill: run only the config-2 prefill part (profiling aid)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.workload == "rowlinear":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable":
                              "the row-parallel linear is a multi-GPU collective; the reference arm "
                              "covers the decode-attention workloads"}))
            return
        run_rowlinear_bench(args)
        return
    if args.workload == "c5":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable":
                              "config 5 on CPU is not a bounded sample: the reference arm covers "
                              "the decode-attention workloads"}))
            return
        run_e2e_llama(args)
        return
    wl = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference_arm(args, wl)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: b200attn has no CPU path")
    rank, world, local = dist_setup(args.gpus)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    peaks = load_peaks()

    if args.only == "prefill":
        pf = run_prefill_bench(args, rank, world, device, peaks)
        if rank == 0:
            print(json.dumps({"only": "prefill", "prefill": pf}))
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    r = run_decode_bench(args, wl, rank, world, device)
    del r["w"], r["out"]
    torch.cuda.empty_cache()
    prefill = None if args.no_prefill else run_prefill_bench(args, rank, world, device, peaks)
    chunks = None
    extras = {}
    if not args.no_extras and args.workload == "c4":
        chunks = run_chunk_bench(args, rank, world, device, peaks)
        for name in ("c1", "c3"):
            x = run_decode_bench(args, WORKLOADS[name], rank, world, device, light=True)
            gbs = x["full_bytes"] / (x["ms_per_step"] * 1e-3) / 1e9
            extras[name] = {"workload": WORKLOADS[name]["desc"],
                            "ms_per_step": round(x["ms_per_step"], 4),
                            "decode_attn_hbm_gbs": round(gbs, 1), "num_splits": x["splits"],
                            "frac_of_hbm_peak": round(gbs / (peaks["hbm_gbs"] * world), 4),
                            "timing": "CUDA-graph replays of the decode step, device events"}
            del x
            torch.cuda.empty_cache()
        if world > 1:
            extras["rowlinear"] = measure_rowlinear(args, rank, world, device)
    elif args.workload == "c3":
        chunks = run_chunk_bench(args, rank, world, device, peaks)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and "kv_dtype" not in wl:
        cpu = run_cpu_baseline(wl)
    e2e_model = e2e_model_fused = None
    if not args.no_e2e_model and args.workload == "c4":
        # the engine gets the GPUs to itself: this process keeps only its CUDA context
        torch.cuda.empty_cache()
        barrier(world)
        e2e_model = run_e2e_model_subprocess(args, rank, world)
        barrier(world)
        # from four ranks up, the same run with o_proj / down_proj through the fused GEMM +
        # all-reduce launch (opt-in in the plugin), so the scaling record holds both
        if world >= 4 and not args.fused_linear:
            args.fused_linear = True
            e2e_model_fused = run_e2e_model_subprocess(args, rank, world, port_offset=41)
            args.fused_linear = False
            barrier(world)

    if rank == 0:
        value = r["full_bytes"] / (r["ms_per_step"] * 1e-3) / 1e9
        e2e = r["full_bytes"] / (r["e2e_ms"] * 1e-3) / 1e9
        achieved = r["rank_bytes"] / (r["decode_ms"] * 1e-3) / 1e9
        traffic = int(r["rank_bytes"] * NCU_READ_PER_ALGORITHMIC_BYTE
                      + r["partial_bytes"] * NCU_WRITE_PER_PARTIAL_BYTE)
        config = workload_config(wl, world, parallelism=f"kv_head_shard{world}")
        config.update({
            "num_splits": r["splits"],
            "step": "one launch: the split-KV decode kernel writes the new K/V rows, streams the "
                    "cache and merges its splits; replayed as one CUDA graph",
            "eager_ms_per_step": round(r["eager_ms_per_step"], 4),
            "l2": "inputs larger than L2 (per-rank KV stream "
                  f"{r['rank_bytes'] / 1e6:.0f} MB vs 126 MB)"})
        line = {
            "metric": "decode_attn_hbm_gbs", "value": round(value, 1), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(r["ms_per_step"], 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config,
            "clocks": r["clocks"],
            "sustained": r.get("sustained"),
            "parity_check": r["parity_check"],
            "e2e": {"value": round(e2e, 1), "unit": "GB/s", "h2d_bytes_per_step": r["h2d"] * world,
                    "d2h_bytes_per_step": r["d2h"] * world, "ms_per_step": round(r["e2e_ms"], 4),
                    "form": "B200AttentionBackendImpl.forward between one pinned host-to-device "
                            "copy of the step's inputs and the device-to-host copy of its output, "
                            "captured once and replayed as a CUDA graph; the host waits for every "
                            "step's output",
                    "eager_ms_per_step": round(r["e2e_eager_ms"], 4),
                    "readback_matches_device": r["e2e_readback_matches"]},
            "gpu_launches": r["launches"],
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                         "traffic": None if "kv_dtype" in wl else traffic,
                         "traffic_source": "not captured for the fp8 kernel" if "kv_dtype" in wl
                         else "constant ratios from one ncu capture of the c4s workload, scaled "
                              "to this launch (not measured in this run)",
                         "peak_source": peaks["source"],
                         "kernel": ("paged_decode_fp8_kernel" if "kv_dtype" in wl
                                    else "paged_decode_splitkv_kernel"),
                         "ms_per_launch": round(r["decode_ms"], 4),
                         "algorithmic_bytes_per_launch": r["rank_bytes"]},
            "cpu_baseline": cpu,
        }
        if prefill:
            line["prefill"] = prefill
        if chunks:
            line["prefill_chunks"] = chunks
        if extras:
            line["extra_workloads"] = extras
        if e2e_model is not None:
            line["e2e_model"] = e2e_model
        if e2e_model_fused is not None:
            line["e2e_model_fused_linear"] = e2e_model_fused
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not r["parity_check"]["ok"]:
        raise SystemExit(f"parity check failed: {r['parity_check']}")


if __name__ == "__main__":
    main()
