"""Row-parallel linear with fused all-reduce (`b200attn_rowlinear_allreduce`) on ONE GPU.

The peers are emulated without a second kernel: before the launch the test itself writes the
peers' fp32 partial sums and their flags (the epoch the call will use) into this rank's
communicator buffer, so the kernel under test never waits for another launch; what it pushes is
read back from the "peer" buffers, which are just other tensors on the same GPU.  The check is
fp32 torch arithmetic on the same bf16 inputs: the kernel accumulates in fp32 and rounds once, so
max |diff| <= one bf16 ulp of the result.  The two-process test on two GPUs lives in
tests/multi_gpu/."""
import pytest
import torch

from oracle.inputs import randn_bf16

pytestmark = pytest.mark.gpu

STAGE_OFF, TILE = 32768, 128


def _bf16_bits(x):
    return x.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF


def _area(buf, world, parity, src, area_bytes):
    """Staging area `src` of one parity: 0..world-1 hold the ranks' partials, `world` results."""
    off = STAGE_OFF + (parity * (world + 1) + src) * area_bytes
    return buf[off:off + area_bytes].view(torch.int32)


def _owner_maps(tokens, n, rows, splits, world):
    """Owner rank (two-shot mode: slot % world, slot = tile * splits + share) of every
    (token, column) and of every (token pair, column)."""
    share = rows // splits
    tile = torch.arange(n, device="cuda") // TILE
    tok = torch.arange(tokens, device="cuda")
    pair_tok = torch.arange((tokens + 1) // 2, device="cuda") * 2
    own_t = (tile[None, :] * splits + (tok // share)[:, None]) % world
    own_p = (tile[None, :] * splits + (pair_tok // share)[:, None]) % world
    return own_t, own_p


def _write_units(area, partial, rows, splits, epoch, slot_mask=None):
    """Lays a [tokens, n] matrix out as the kernel expects to find it: units
    {bf16(t) | bf16(t+1) << 16, epoch} at [tile * splits + share][pair][column].  `slot_mask`
    [tiles, splits] limits the write to some slots."""
    tokens, n = partial.shape
    tiles = (n + TILE - 1) // TILE
    share = rows // splits
    padded = torch.zeros(rows, tiles * TILE, device=partial.device)
    padded[:tokens, :n] = partial
    bits = _bf16_bits(padded).view(splits, share // 2, 2, tiles, TILE)
    data = bits[:, :, 0] | (bits[:, :, 1] << 16)                     # [splits, pairs, tiles, col]
    units = torch.stack([data, torch.full_like(data, epoch)], dim=-1)
    units = units.permute(2, 0, 1, 3, 4).contiguous()                # [tiles, splits, pairs, col, 2]
    if slot_mask is None:
        area[:units.numel()] = units.view(-1)
    else:
        view = area[:units.numel()].view(units.shape)
        view[slot_mask] = units[slot_mask]


def _read_units(area, tokens, n, rows, splits):
    """Inverse of _write_units: (bf16 values as fp32 [tokens, n], flags [tokens // 2.., n])."""
    tiles = (n + TILE - 1) // TILE
    share = rows // splits
    units = area[:tiles * rows // 2 * TILE * 2].view(tiles, splits, share // 2, TILE, 2)
    data, flags = units[..., 0], units[..., 1]
    lo = (data << 16).view(torch.float32)
    hi = (data & -65536).view(torch.float32)
    vals = torch.stack([lo, hi], dim=3)                               # [tiles, splits, pairs, 2, col]
    vals = vals.permute(1, 2, 3, 0, 4).reshape(rows, tiles * TILE)
    flags = flags.permute(1, 2, 0, 3).reshape(rows // 2, tiles * TILE)
    return vals[:tokens, :n], flags[:(tokens + 1) // 2, :n]


def _close(out, ref_fp32, what, scale=None):
    ref = ref_fp32.float()
    err = (out.float() - ref).abs()
    mag = ref.abs() if scale is None else scale
    tol = mag * 2 ** -6 + 1e-3          # two bf16 ulps of the magnitude, plus a floor
    assert bool((err <= tol).all()), f"{what}: max err {err.max().item():.4g}"


@pytest.mark.parametrize("tokens,n,k", [(64, 4096, 2048), (1, 4096, 512), (128, 4096, 1024),
                                        (37, 1024, 7168), (64, 8192, 256), (5, 96, 72)])
def test_single_rank_is_a_plain_gemm(tokens, n, k, clean_error_word):
    from b200attn import tp_linear

    g = torch.Generator().manual_seed(tokens + n + k)
    x = randn_bf16((tokens, k), g).cuda()
    w = (randn_bf16((n, k), g) * 0.05).to(torch.bfloat16).cuda()
    out = tp_linear.rowlinear_allreduce(x, w, None)
    _close(out, x.float() @ w.float().T, f"gemm {tokens}x{n}x{k}")


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 2), (8, 7)])
@pytest.mark.parametrize("tokens,n,k", [(64, 4096, 512), (3, 256, 128), (128, 1024, 2048),
                                        (33, 200, 64)])
@pytest.mark.parametrize("mode", [1, 2])
def test_fused_allreduce_with_emulated_peers(mode, world, rank, tokens, n, k, clean_error_word):
    """mode 1: one shot (every peer's partial is found in this rank's areas, its own partial is
    pushed to every peer).  mode 2: two shots (for the slots this rank owns it finds every peer's
    partial and pushes the result to every peer; for the others it pushes its partial to the
    owner only and finds the owner's result)."""
    from b200attn import tp_linear

    g = torch.Generator().manual_seed(world * 10 + rank + tokens)
    max_tokens, max_n = 128, 4096
    nbytes = tp_linear.comm_bytes(world, max_tokens, max_n)
    ab = tp_linear.area_bytes(max_tokens, max_n)
    assert nbytes == STAGE_OFF + 2 * (world + 1) * ab
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    comm = tp_linear.RowLinearComm(buffers=bufs, rank=rank, max_n=max_n, max_tokens=max_tokens)
    hdr = bufs[rank][:8].view(torch.int32)
    rows, splits = tp_linear.plan(tokens, n, k)
    tiles = (n + TILE - 1) // TILE
    slot_owner = (torch.arange(tiles * splits, device="cuda") % world).view(tiles, splits)
    own_t, own_p = _owner_maps(tokens, n, rows, splits, world)
    w = (randn_bf16((n, k), g) * 0.05).to(torch.bfloat16).cuda()
    for call in (1, 2, 3):                      # epochs 1, 2, 3: both staging parities, reuse
        x = randn_bf16((tokens, k), g).cuda()
        mine = x.float() @ w.float().T
        partials = [torch.randn(tokens, n, generator=g).cuda() for _ in range(world)]
        partials[rank] = mine
        want = torch.zeros_like(mine)
        mag = torch.zeros_like(mine)
        for src in range(world):                # rank order, bf16 partials, like the kernel
            want = want + partials[src].to(torch.bfloat16).float()
            mag = mag + partials[src].abs()
        mask_mine = None if mode == 1 else slot_owner == rank
        for src in range(world):
            if src != rank:
                _write_units(_area(bufs[rank], world, call & 1, src, ab), partials[src], rows,
                             splits, call, mask_mine)
        if mode == 2:                           # the owners' results for the slots of the others
            _write_units(_area(bufs[rank], world, call & 1, world, ab), want, rows, splits, call,
                         slot_owner != rank)
        torch.cuda.synchronize()
        out = tp_linear.rowlinear_allreduce(x, w, comm, peer_timeout_s=0.5, reduce_mode=mode)
        torch.cuda.synchronize()
        _close(out, want, f"call {call}", scale=mag)
        assert int(hdr[0]) == call and int(hdr[1]) == 0          # epoch published, ticket reset
        for peer in range(world):
            if peer == rank:
                continue
            vals, flags = _read_units(_area(bufs[peer], world, call & 1, rank, ab), tokens, n,
                                      rows, splits)
            # partial pushed to `peer`: always in one-shot mode, only where `peer` owns the slot
            sent_p = torch.ones_like(own_p, dtype=torch.bool) if mode == 1 else own_p == peer
            sent_t = torch.ones_like(own_t, dtype=torch.bool) if mode == 1 else own_t == peer
            assert bool((flags[sent_p] == call).all()) and bool((flags[~sent_p] != call).all())
            _close(vals[sent_t], mine[sent_t], "pushed partial")
            if mode == 2:                       # results of this rank's slots go to every peer
                res, rflags = _read_units(_area(bufs[peer], world, call & 1, world, ab), tokens,
                                          n, rows, splits)
                assert bool((rflags[own_p == rank] == call).all())
                assert bool((rflags[own_p != rank] != call).all())
                assert torch.equal(res[own_t == rank], out.float()[own_t == rank])


def test_missing_peer_times_out_and_reports(clean_error_word):
    """A peer that never arrives: the bounded wait runs out, the diagnostics word says so, the
    context stays usable and later launches return at once until the word is read."""
    from b200attn import ops, tp_linear

    g = torch.Generator().manual_seed(1)
    nbytes = tp_linear.comm_bytes(2, 16, 256)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    comm = tp_linear.RowLinearComm(buffers=bufs, rank=0, max_n=256, max_tokens=16)
    x = randn_bf16((4, 128), g).cuda()
    w = randn_bf16((256, 128), g).cuda()
    tp_linear.rowlinear_allreduce(x, w, comm, peer_timeout_s=0.05)
    torch.cuda.synchronize()
    assert ops.read_error_word() == 1
    # the GPU still works
    out = tp_linear.rowlinear_allreduce(x, w, None)
    _close(out, x.float() @ w.float().T, "after timeout")
    assert ops.read_error_word() == 0


def test_argument_checks():
    from b200attn import tp_linear

    x = torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(64, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="expected"):
        tp_linear.rowlinear_allreduce(x, w[:, :64], None)
    with pytest.raises(ValueError, match="bfloat16"):
        tp_linear.rowlinear_allreduce(x.float(), w.float(), None)
    with pytest.raises(RuntimeError, match="maximum"):
        tp_linear.rowlinear_allreduce(torch.zeros(129, 128, dtype=torch.bfloat16, device="cuda"), w,
                                      None)
    with pytest.raises(RuntimeError, match="no CPU path"):
        tp_linear.rowlinear_allreduce(x.cpu(), w.cpu(), None)
    with pytest.raises(ValueError, match="geometry"):
        tp_linear.comm_bytes(9, 64, 4096)
