"""The one-launch GPU metadata builder against the host statement of the runner's arithmetic, and
driving a forward pass with the metadata it produced."""
import pytest
import torch

from b200attn import metadata as md
from oracle import restate
from oracle.inputs import randn_bf16
from tests.conftest import assert_attention_close

pytestmark = pytest.mark.gpu


def _device_out(rows, width, fill_width, tokens_per_row):
    # pre-filled with junk: the builder must overwrite every entry of the persistent buffers
    return md.StepMetadata(
        torch.full((rows,), 77, dtype=torch.int32, device="cuda"),
        torch.full((rows, width), 77, dtype=torch.int32, device="cuda"),
        torch.full((rows, fill_width), 77, dtype=torch.int32, device="cuda"),
        torch.full((rows * tokens_per_row,), 77, dtype=torch.int64, device="cuda"), None)


@pytest.mark.parametrize("tokens_per_row,bs", [(1, 32), (1, 64), (64, 32), (256, 64)])
def test_builder_matches_host(tokens_per_row, bs):
    g = torch.Generator().manual_seed(tokens_per_row + bs)
    n, rows, width = 13, 16, 40
    fill_width = md.fill_page_table_width(tokens_per_row, bs, width)
    bt = (torch.randperm(n * width, generator=g) + 1).reshape(n, width).int()
    if tokens_per_row == 1:
        computed = torch.randint(0, width * bs - 1, (n,), generator=g).int()
        sched = torch.ones(n, dtype=torch.int32)
    else:
        computed = torch.full((n,), 3 * bs, dtype=torch.int32)     # one shared chunk start
        sched = torch.randint(1, tokens_per_row + 1, (n,), generator=g).int()
    sched[4] = 0                                                   # a parked row
    want = md.build_step_metadata_host(computed, sched, bt, bs, rows, tokens_per_row, fill_width)
    out = _device_out(rows, width, fill_width, tokens_per_row)
    md.build_step_metadata(computed.cuda(), sched.cuda(), bt.cuda(), bs, out, tokens_per_row)
    assert torch.equal(out.cache_position.cpu(), want.cache_position)
    assert torch.equal(out.page_table.cpu(), want.page_table)
    assert torch.equal(out.fill_page_table.cpu(), want.fill_page_table)
    assert torch.equal(out.slot_mapping.cpu(), want.slot_mapping)


def test_decode_step_driven_by_device_built_metadata(clean_error_word):
    """Scheduler state stays on the device: builder -> forward, checked against the oracle."""
    from b200attn import B200AttentionBackendImpl, B200Metadata

    g = torch.Generator().manual_seed(5)
    nq, nkv, hd, bs, n, rows, width = 16, 4, 128, 64, 6, 8, 12
    bt = (torch.randperm(n * width, generator=g) + 1).reshape(n, width).int()
    computed = torch.randint(1, width * bs - 1, (n,), generator=g).int()
    sched = torch.ones(n, dtype=torch.int32)
    nb = n * width + 1
    kc = randn_bf16((nb, nkv, bs, hd), g)
    vc = randn_bf16((nb, nkv, bs, hd), g)
    q = randn_bf16((rows, nq * hd), g)
    k = randn_bf16((rows, nkv * hd), g)
    v = randn_bf16((rows, nkv * hd), g)
    out_md = _device_out(rows, width, 8, 1)
    md.build_step_metadata(computed.cuda(), sched.cuda(), bt.cuda(), bs, out_md, 1)
    impl = B200AttentionBackendImpl(nq, hd, hd ** -0.5, nkv, None, None, "auto")
    meta = B200Metadata(cache_position=out_md.cache_position, page_table=out_md.page_table,
                        fill_page_table=out_md.fill_page_table, num_users=rows,
                        batch_idx=torch.arange(rows, dtype=torch.int32, device="cuda"))
    kv = [kc.cuda(), vc.cuda()]
    out = torch.empty(rows, nq * hd, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, q.cuda(), k.cuda(), v.cuda(), kv, meta, output=out)
    pos = computed + sched - 1
    want_out, want_k, want_v = restate.impl_forward(
        q[:n], k[:n], v[:n], kc, vc, num_heads=nq, num_kv_heads=nkv, head_size=hd,
        scale=hd ** -0.5, num_users=n, cache_position=pos, page_table=bt,
        compute_dtype=torch.float32)
    # padded rows (cache_position -1, null page table) write into the null block 0 only
    got_k, got_v = kv[0].cpu(), kv[1].cpu()
    assert torch.equal(got_k[1:], want_k[1:]) and torch.equal(got_v[1:], want_v[1:])
    assert_attention_close(out[:n], want_out, "decode via device-built metadata")
    assert out[n:].abs().sum().item() == 0


def test_device_step_state_drives_two_steps_on_the_same_buffers(clean_error_word):
    """The product path of the builder: scheduler state on the device, one launch per step into
    persistent buffers, the Impl's forward on the result; two steps in a row (the second one
    more token into every context)."""
    from b200attn import B200AttentionBackendImpl, B200AttentionMetadataBuilder

    g = torch.Generator().manual_seed(15)
    nq, nkv, hd, bs, n, rows, width = 8, 2, 64, 32, 5, 8, 10
    bt = (torch.randperm(n * width, generator=g) + 1).reshape(n, width).int()
    computed = torch.randint(1, width * bs - 3, (n,), generator=g).int()
    sched = torch.ones(n, dtype=torch.int32)
    nb = n * width + 1
    kc, vc = randn_bf16((nb, nkv, bs, hd), g), randn_bf16((nb, nkv, bs, hd), g)
    state = B200AttentionMetadataBuilder(device=torch.device("cuda")).device_step_state(
        rows, width, bs, tokens_per_row=1)
    impl = B200AttentionBackendImpl(nq, hd, hd ** -0.5, nkv, None, None, "auto")
    kv = [kc.cuda(), vc.cuda()]
    d_computed, d_sched, d_bt = computed.cuda(), sched.cuda(), bt.cuda()
    ptrs = None
    for step in range(2):
        q, k, v = (randn_bf16((rows, h * hd), g) for h in (nq, nkv, nkv))
        meta = state.build(d_computed, d_sched, d_bt)
        now = (meta.cache_position.data_ptr(), meta.page_table.data_ptr())
        assert ptrs is None or now == ptrs           # same buffers every step
        ptrs = now
        out = torch.empty(rows, nq * hd, dtype=torch.bfloat16, device="cuda")
        impl.forward(None, q.cuda(), k.cuda(), v.cuda(), kv, meta, output=out)
        want_out, kc, vc = restate.impl_forward(
            q[:n], k[:n], v[:n], kc, vc, num_heads=nq, num_kv_heads=nkv, head_size=hd,
            scale=hd ** -0.5, num_users=n, cache_position=computed + sched - 1, page_table=bt,
            compute_dtype=torch.float32)
        assert torch.equal(kv[0].cpu()[1:], kc[1:]) and torch.equal(kv[1].cpu()[1:], vc[1:])
        assert_attention_close(out[:n], want_out, f"step {step}")
        assert out[n:].abs().sum().item() == 0
        computed = computed + 1
        d_computed += 1
