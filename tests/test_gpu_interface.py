"""The FlashMLA-shaped surface (flash_mla_sm120/interface.py:35-194) against the CPU oracle."""
import pytest
import torch

import helpers as H
from helpers import make_case, oracle_attn

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _check(out, lse_bhs, ref_out, ref_lse, b, s_q):
    heads = ref_out.shape[1]
    assert out.shape == (b, s_q, heads, 512) and out.dtype == torch.bfloat16
    assert lse_bhs.shape == (b, heads, s_q) and lse_bhs.dtype == torch.float32
    H.compare_out(out.reshape(b * s_q, heads, 512).cpu(), ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)
    lse_tok = lse_bhs.permute(0, 2, 1).reshape(b * s_q, heads).cpu()
    H.compare_lse(lse_tok, ref_lse, H.TC_LSE)


@pytest.mark.parametrize("b,s_q,topk", [(3, 2, 256), (1, 1, 512), (70, 1, 128)])
def test_with_kvcache_shapes_and_values(b, s_q, topk):
    """s_q query tokens per request are flattened; one token takes the split path (more
    partitions than tokens), 70 tokens the unsplit one."""
    from sparse_mla_sm120_b200 import interface
    case = make_case(31, b * s_q, 128, topk, 16)
    ref_out, ref_lse = oracle_attn(case)
    q = case["q"].view(b, s_q, 128, 576).to(DEV)
    kv = case["packed"].to(DEV)
    idx = case["indices"].view(b, s_q, topk).to(DEV)
    meta, none = interface.get_mla_metadata()
    assert none is None and not meta.have_initialized
    out, lse = interface.flash_mla_with_kvcache(q, kv, None, None, 512, meta, None, case["sm_scale"], False, True,
                                                indices=idx)
    _check(out, lse, ref_out, ref_lse, b, s_q)
    assert meta.have_initialized and meta.config.b == b and meta.config.s_q == s_q and meta.config.topk == topk
    # a second layer of the same step reuses the metadata and gives the same result
    out2, lse2 = interface.flash_mla_with_kvcache(q, kv, None, None, 512, meta, None, case["sm_scale"], False, True,
                                                  indices=idx)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    # a different configuration with the same object is refused
    with pytest.raises(ValueError):
        interface.flash_mla_with_kvcache(q, kv, None, None, 512, meta, None, case["sm_scale"], False, True,
                                         indices=idx[..., : topk // 2].contiguous())


def test_sparse_fwd_accepts_3d_indices():
    from sparse_mla_sm120_b200 import interface
    case = make_case(32, 5, 64, 192, 8)
    ref_out, ref_lse = oracle_attn(case)
    out, mx, lse = interface.flash_mla_sparse_fwd(case["q"].to(DEV), case["packed"].to(DEV),
                                                  case["indices"].unsqueeze(1).to(DEV), case["sm_scale"])
    H.compare_out(out.cpu(), ref_out, H.TC_PREFILL_ABS, H.TC_PREFILL_REL, H.TC_COS)
    H.compare_lse(lse.cpu(), ref_lse, H.TC_LSE)
    assert mx.shape == (5, 64)
