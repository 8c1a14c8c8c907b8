"""The hand-over of a norm to the projections around it, as far as it is
decided on the host: who is offered a sink, who gets an unscaled norm output,
and what a norm refuses. No kernel runs here."""
import pytest
import torch

from foundry_b200.kernels import ops
from foundry_b200.parts.block import _sink_for
from foundry_b200.parts.norm import RMSNorm


def norm_of(dtype, size=8):
    norm = RMSNorm(size, 1e-5, dtype=dtype, device=torch.device("cpu"))
    norm.weight = torch.ones(size)
    return norm


class Accepting:
    accepts_row_scaled = True


class Plain:
    pass


class NormWithoutSink:
    pass


def test_a_sink_is_offered_only_in_front_of_a_part_that_takes_unscaled_rows():
    resid = torch.zeros(2, 8)
    norm = norm_of(torch.bfloat16)
    sink = _sink_for(norm, Accepting(), resid)
    assert isinstance(sink, ops.ResidualSink)
    assert sink.resid is resid and sink.gamma is norm.weight and sink.eps == norm.eps
    assert _sink_for(norm, Plain(), resid) is None
    assert _sink_for(NormWithoutSink(), Accepting(), resid) is None


def test_a_32_bit_norm_or_one_without_weights_offers_no_sink():
    resid = torch.zeros(2, 8)
    assert norm_of(torch.float32).sink(resid) is None
    unloaded = RMSNorm(8, 1e-5, dtype=torch.bfloat16, device=torch.device("cpu"))
    assert unloaded.sink(resid) is None


def test_the_norm_turns_its_own_pending_result_into_unscaled_rows():
    resid = torch.zeros(2, 8)
    norm = norm_of(torch.bfloat16)
    values, shares = torch.zeros(2, 8, dtype=torch.bfloat16), torch.zeros(1, 16)
    pending = ops.NormPending(norm.sink(resid), values, shares)
    scaled = norm.add_norm(resid, pending)
    assert isinstance(scaled, ops.RowScaled)
    assert scaled.values is values and scaled.shares is shares and scaled.eps == norm.eps
    assert scaled.shape == values.shape and scaled.dtype == torch.bfloat16
    assert ops.plain(values) is values  # a tensor stays what it is


def test_a_pending_result_made_for_other_rows_or_another_norm_is_refused():
    resid, other = torch.zeros(2, 8), torch.zeros(2, 8)
    norm, second = norm_of(torch.bfloat16), norm_of(torch.bfloat16)
    values, shares = torch.zeros(2, 8, dtype=torch.bfloat16), torch.zeros(1, 16)
    pending = ops.NormPending(norm.sink(resid), values, shares)
    with pytest.raises(ops.KernelError, match="another"):
        norm.add_norm(other, pending)
    with pytest.raises(ops.KernelError, match="another"):
        second.add_norm(resid, pending)
