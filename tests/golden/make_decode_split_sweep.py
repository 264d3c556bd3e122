"""Measures the decode launch for a set of batch shapes at several split counts on the GPU at
hand and writes tests/golden/decode_split_sweep.json: the data the split-count cost model
(`b200attn_decode_auto_splits`) is fitted to and that tests/test_split_model.py holds it against.

    python tests/golden/make_decode_split_sweep.py          # needs a B200 and the built library

Per shape and split count: ten decode calls captured into one CUDA graph, five timed replays by
CUDA events (L2 flushed between replays when the K/V stream is smaller than L2), median, in
microseconds per call.  Contexts are drawn uniformly from [lo, hi] with a fixed seed; `hint` is
the `max_context_len` the caller would pass."""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tt-xla_b200"))
from b200attn import ops  # noqa: E402

SHAPES = [
    # name, users, nq, nkv, hd, bs, ctx lo, ctx hi, split counts, hint
    ("c5 B64 ctx~1150 hint2048", 64, 32, 8, 128, 64, 1024, 1280, [1, 2, 3, 4, 6, 8], 2048),
    ("c5 TP2", 64, 16, 4, 128, 64, 1024, 1280, [1, 2, 3, 4, 6, 8], 2048),
    ("c5 TP4", 64, 8, 2, 128, 64, 1024, 1280, [1, 2, 3, 4, 6, 8], 2048),
    ("c5 TP8 B64 nkv1", 64, 4, 1, 128, 64, 1024, 1280, [1, 2, 4, 6, 8, 16], 2048),
    ("c3 B64 ctx1k-8k", 64, 32, 8, 128, 64, 1024, 8192, [1, 2, 3, 4, 6, 8, 12], 8192),
    ("c3 TP2", 64, 16, 4, 128, 64, 1024, 8192, [1, 2, 3, 4, 6, 8, 12], 8192),
    ("c3 TP4", 64, 8, 2, 128, 64, 1024, 8192, [1, 2, 3, 4, 6, 8, 12, 16], 8192),
    ("c3 TP8 nkv1", 64, 4, 1, 128, 64, 1024, 8192, [2, 3, 4, 6, 8, 12, 16], 8192),
    ("c4s B8 ctx8192", 8, 64, 8, 128, 64, 8192, 8192, [2, 3, 4, 6, 8, 16], 8192),
    ("c4 B32 ctx32768", 32, 64, 8, 128, 64, 32768, 32768, [1, 2, 3, 4, 6, 8, 16], 32768),
    ("c4 TP2 nkv4", 32, 32, 4, 128, 64, 32768, 32768, [1, 2, 3, 4, 6, 8, 12, 16], 32768),
    ("c4 TP4 nkv2", 32, 16, 2, 128, 64, 32768, 32768, [2, 3, 4, 6, 8, 12, 16], 32768),
    ("c4 TP8 nkv1", 32, 8, 1, 128, 64, 32768, 32768, [4, 6, 8, 9, 12, 16, 24], 32768),
    ("c1 B8 hd64", 8, 32, 8, 64, 32, 128, 1024, [1, 2, 3, 4, 6, 8, 16], 1024),
    ("c1 TP8 nkv1", 8, 4, 1, 64, 32, 128, 1024, [1, 2, 4, 8, 16], 1024),
    ("B1 ctx 8192", 1, 32, 8, 128, 64, 8192, 8192, [4, 8, 12, 16, 24, 32, 64], 8192),
    ("B1 ctx 131072 nkv8", 1, 32, 8, 128, 64, 131072, 131072, [8, 12, 16, 24, 37, 64], 131072),
    ("B16 ctx 4096 nkv8", 16, 32, 8, 128, 64, 4096, 4096, [1, 2, 3, 4, 6, 8], 4096),
    ("B128 ctx 2048 nkv8", 128, 32, 8, 128, 64, 2048, 2048, [1, 2, 3, 4], 2048),
    ("B4 ctx 16384 nkv2 hd64", 4, 8, 2, 64, 32, 16384, 16384, [8, 16, 24, 32, 48, 64, 96], 16384),
]


def measure(name, users, nq, nkv, hd, bs, lo, hi, splits_list, hint, flush):
    g = torch.Generator().manual_seed(0)
    ctx = torch.randint(lo, hi + 1, (users,), generator=g)
    nblk = (hi + bs - 1) // bs
    nb = users * nblk
    page_table = torch.randperm(nb, generator=g).reshape(users, nblk).int().cuda()
    kc = torch.randn(nb, nkv, bs, hd, device="cuda").bfloat16()
    vc = torch.randn(nb, nkv, bs, hd, device="cuda").bfloat16()
    q = torch.randn(users, nq, hd, device="cuda").bfloat16()
    out = torch.empty_like(q)
    pos = (ctx - 1).int().cuda()
    kv_bytes = int(ctx.sum()) * 2 * nkv * hd * 2
    reps = 10
    row = dict(name=name, users=users, nkv=nkv, hd=hd, hint=hint,
               mean_ctx=round(float(ctx.float().mean()), 1), times={})
    for s in splits_list:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ops.paged_decode(q, kc, vc, page_table, pos, out=out, num_splits=s, max_context_len=hint)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(reps):
                ops.paged_decode(q, kc, vc, page_table, pos, out=out, num_splits=s,
                                 max_context_len=hint)
        for _ in range(3):
            graph.replay()
        ts = []
        for _ in range(5):
            if kv_bytes < (200 << 20):
                flush.zero_()
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / reps)
        row["times"][str(s)] = round(sorted(ts)[len(ts) // 2] * 1e3, 2)
    return row


def main():
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    for shape in SHAPES:
        rows.append(measure(*shape, flush))
        print(rows[-1]["name"], rows[-1]["times"], flush=True)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "decode_split_sweep.json")
    with open(path, "w") as f:
        json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
