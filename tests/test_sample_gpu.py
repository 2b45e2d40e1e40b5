"""Sampling tail (top-p cut and one draw per row) over the survivors of the fused operator: the GPU choice
must be the oracle's, position for position, because both sum sequentially in fp32."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from tests import util
from vkop_b200 import workloads

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from vkop_b200 import capi as c
    return c


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("top_p", [1.0, 0.9, 0.5, 0.01])
def test_sampling_matches_the_oracle(capi, dtype, top_p):
    x = workloads.llm_vocab(seed=31, rows=64).to(dtype)
    vals, idx = capi.softmax_topk(x.cuda(), 50, 1.25)
    g = torch.Generator().manual_seed(9)
    u = torch.rand(64, generator=g)
    u[0], u[1] = 0.0, 0.99999994  # both ends of [0, 1)
    choice, token = capi.sample_topk(vals, idx, top_p, u.cuda())
    torch.cuda.synchronize()
    want_choice, want_token = oracle.sample_topk(util.to_oracle_array(vals.cpu()), idx.cpu().numpy(), top_p, u.numpy(),
                                                 dtype=util.ORACLE_DTYPE[dtype])
    assert np.array_equal(choice.cpu().numpy(), want_choice)
    assert np.array_equal(token.cpu().numpy().astype(np.int64), want_token)
    assert (choice >= 0).all() and (choice < 50).all()
    if top_p <= 0.01:
        assert (choice == 0).all()  # the nucleus is the best candidate alone


def test_sampling_int64_and_distribution(capi):
    # a known distribution, many draws: frequencies follow the renormalised nucleus
    p = torch.tensor([0.4, 0.3, 0.2, 0.1]).repeat(20000, 1).cuda()
    ids = torch.tensor([11, 22, 33, 44], dtype=torch.int64).repeat(20000, 1).cuda()
    u = torch.rand(20000, generator=torch.Generator().manual_seed(3)).cuda()
    choice, token = capi.sample_topk(p, ids, 0.85, u)  # nucleus = first three (0.9 >= 0.85)
    torch.cuda.synchronize()
    assert token.dtype == torch.int64
    freq = torch.bincount(choice.long().cpu(), minlength=4).float() / 20000
    assert freq[3] == 0
    assert torch.allclose(freq[:3], torch.tensor([0.4, 0.3, 0.2]) / 0.9, atol=0.015)
    assert torch.equal(token.cpu(), torch.tensor([11, 22, 33, 44])[choice.long().cpu()])


def test_sampling_argument_errors(capi):
    v = torch.rand(2, 4).cuda()
    i = torch.zeros(2, 4, dtype=torch.int32).cuda()
    u = torch.rand(2).cuda()
    with pytest.raises(capi.VkopError):
        capi.sample_topk(v, i, 0.0, u)
