"""Host-side logic of the fused row-parallel linear (no GPU): which calls take the fused launch,
argument checks, staging geometry arithmetic."""
import pytest
import torch

from b200attn import tp_linear


class FakeComm:
    max_tokens, max_n, world, rank = 128, 4096, 2, 0


class FakeRowParallel(torch.nn.Module):
    """Stand-in with the attributes of vLLM's RowParallelLinear that the dispatch looks at."""

    def __init__(self, n=256, k=64, bias=False, dtype=torch.bfloat16):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.zeros(n, k, dtype=dtype), requires_grad=False)
        self.bias = torch.nn.Parameter(torch.zeros(n, dtype=dtype)) if bias else None
        self.reduce_results = True
        self.input_is_parallel = True
        self.return_bias = True
        self.calls = 0

    def forward(self, x):
        self.calls += 1
        return "original", None


def test_dispatch_keeps_the_original_forward_outside_the_fused_case(monkeypatch):
    fused_calls = []
    monkeypatch.setattr(tp_linear, "rowlinear_allreduce",
                        lambda x, w, comm: fused_calls.append(tuple(x.shape)) or "fused")
    comm = FakeComm()
    layer = tp_linear.partition_row_parallel_linear(FakeRowParallel(), comm)
    bf = torch.bfloat16
    assert layer.forward(torch.zeros(64, 64, dtype=bf)) == ("fused", None)
    assert layer.forward(torch.zeros(128, 64, dtype=bf)) == ("fused", None)
    assert layer.forward(torch.zeros(129, 64, dtype=bf))[0] == "original"       # too many rows
    assert layer.forward(torch.zeros(0, 64, dtype=bf))[0] == "original"         # empty batch
    assert layer.forward(torch.zeros(4, 64))[0] == "original"                   # fp32 input
    assert layer.forward(torch.zeros(2, 4, 64, dtype=bf))[0] == "original"      # not 2-D
    assert fused_calls == [(64, 64), (128, 64)]
    layer.return_bias = False
    assert layer.forward(torch.zeros(8, 64, dtype=bf)) == "fused"
    # bias, unreduced output, replicated input and wide outputs keep the layer's own forward
    for kw in (dict(bias=True), dict(n=8192)):
        other = tp_linear.partition_row_parallel_linear(FakeRowParallel(**kw), comm)
        assert other.forward(torch.zeros(8, 64, dtype=bf))[0] == "original"
    for attr in ("reduce_results", "input_is_parallel"):
        other = FakeRowParallel()
        setattr(other, attr, False)
        other = tp_linear.partition_row_parallel_linear(other, comm)
        assert other.forward(torch.zeros(8, 64, dtype=bf))[0] == "original"


def test_refuses_cpu_tensors_and_bad_shapes():
    bf = torch.bfloat16
    with pytest.raises(RuntimeError, match="no CPU path"):
        tp_linear.rowlinear_allreduce(torch.zeros(4, 64, dtype=bf), torch.zeros(8, 64, dtype=bf), None)
    with pytest.raises(RuntimeError, match="no CPU path"):
        tp_linear.RowLinearComm(buffers=[torch.zeros(1 << 20, dtype=torch.uint8)] * 2, rank=0,
                                max_n=256, max_tokens=16)


def test_staging_geometry():
    # one area: 8-byte units, one per bf16 pair: tiles * token rows / 2 * 128 columns * 8 bytes
    assert tp_linear.area_bytes(64, 4096) == 32 * 64 * 512
    assert tp_linear.area_bytes(65, 4096) == 32 * 128 * 512
    assert tp_linear.area_bytes(1, 100) == 1 * 32 * 512
    # per parity one area per rank plus one for two-shot results, behind a 32 KiB prefix
    assert tp_linear.comm_bytes(8, 128, 4096) == 32768 + 2 * 9 * tp_linear.area_bytes(128, 4096)
    assert tp_linear.comm_bytes(2, 64, 4096) == 32768 + 2 * 3 * tp_linear.area_bytes(64, 4096)
    for bad in ((0, 64, 4096), (9, 64, 4096), (2, 129, 4096), (2, 0, 4096)):
        with pytest.raises(ValueError, match="geometry"):
            tp_linear.comm_bytes(*bad)
