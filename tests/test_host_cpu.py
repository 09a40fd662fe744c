"""Argument checks of the host-memory step that need no GPU."""
import pytest
import torch

from delta_matching_b200.host import attn_step_host


def test_rejects_wrong_rank_and_dtype():
    x = torch.zeros(2, 256, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        attn_step_host(x[0], x, x, x)
    with pytest.raises(TypeError):
        attn_step_host(x.float(), x, x, x)
    with pytest.raises(ValueError):
        attn_step_host(x.transpose(1, 2), x, x, x)                 # not contiguous
