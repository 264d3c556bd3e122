"""One rank of the multi-GPU check of the fused row-parallel linear (run under torchrun, one
process per GPU; NCCL only carries the comparison data, never the kernel under test).

Every rank draws the SAME full x [tokens, K] and w [N, K] from a shared seed, keeps its K slice,
calls the fused op, and compares with fp32 arithmetic on the full matrices.  All ranks must also
return identical bits.  Prints one line `ROWLINEAR_OK world=<n>` on rank 0 when every case passed."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "tt-xla_b200"))


def main() -> int:
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    from b200attn import ops, tp_linear

    comm = tp_linear.RowLinearComm(dist.group.WORLD, max_n=8192, max_tokens=128)
    ok = True
    cases = [(64, 4096, 4096), (1, 4096, 4096), (128, 4096, 14336), (17, 8192, 1024),
             (64, 4096, 4096)]
    for i, (tokens, n, k_full) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + i)
        x = torch.randn(tokens, k_full, generator=g).to(torch.bfloat16)
        w = (torch.randn(n, k_full, generator=g) * 0.03).to(torch.bfloat16)
        kl = k_full // world
        xs = x[:, rank * kl:(rank + 1) * kl].contiguous().cuda()
        ws = w[:, rank * kl:(rank + 1) * kl].contiguous().cuda()
        mode = (0, 1, 2)[i % 3]                    # automatic, one shot, two shots
        for rep in range(3):                      # back-to-back calls exercise both parities
            out = tp_linear.rowlinear_allreduce(xs, ws, comm, peer_timeout_s=5.0, reduce_mode=mode)
        torch.cuda.synchronize()
        # what every rank must return: its peers' and its own partial products rounded to bf16,
        # added in rank order in fp32 (one more rounding at the end)
        ref = torch.zeros(tokens, n)
        mag = torch.zeros(tokens, n)
        for r in range(world):
            part = (x[:, r * kl:(r + 1) * kl].float() @ w[:, r * kl:(r + 1) * kl].float().T)
            ref += part.to(torch.bfloat16).float()
            mag += part.abs()
        ref, mag = ref.cuda(), mag.cuda()
        err = (out.float() - ref).abs()
        tol = mag * 2 ** -6 + 2e-3     # two bf16 ulps of the summed magnitudes
        good = bool((err <= tol).all())
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        if not (good and same):
            ok = False
            print(f"rank {rank} case {i} {tokens}x{n}x{k_full}: max err {err.max().item():.4g} "
                  f"identical={same}", flush=True)
    word = ops.read_error_word()
    if word != 0:
        ok = False
        print(f"rank {rank}: diagnostics word {word}", flush=True)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag) == 1:
        print(f"ROWLINEAR_OK world={world}", flush=True)
    comm.close()
    dist.destroy_process_group()
    return 0 if int(flag) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
