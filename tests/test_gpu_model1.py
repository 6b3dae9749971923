"""The 584-byte MODEL1 cache layout and the second ("extra") cache on the GPU, against the oracle and the
fixtures made by the reference's own helpers.  Cases follow tests/test_v4_features.py (variable topk_length,
extra cache with and without lengths, sink with +-inf) and tests/test_prefill.py:224-454 of the reference.

Every case runs on both kernels: the exact fp32 kernel (bound: the rounding of the output to bf16) and the
tcgen05 kernel (bound: the FP8-class tolerances of helpers.py, which for this randn/10 data are the reference's own
1e-3 + 2.01/128 form, tests/test_v4_features.py:28-31)."""
import math

import pytest
import torch

import helpers as H
from helpers import orc
from test_oracle_golden import M1_CASES, load_m1_case

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
FP32, TC = 1, 2


@pytest.fixture(params=[FP32, TC], ids=["fp32", "tc"])
def impl(request):
    return request.param


def _dev(t):
    return None if t is None else t.to(DEV)


def _expected_lse(lse, sink):
    """The kernels fold the sink into the LSE they return (decode_v2_kernel.cuh:582-595)."""
    if sink is None:
        return lse.double()
    return torch.logaddexp(lse.double(), sink.double().view(*([1] * (lse.dim() - 1)), -1).expand_as(lse))


def _compare(out, lse2, ref_out, ref_lse, sink=None, impl=FP32, case=None):
    """`case` (tensor-core kernel only): derive the bound from the FP8-class emulation on the same inputs instead of
    the fixed FP8-class tolerances; for cases with random lengths, whose shortest rows average a handful of tokens."""
    if impl == TC and case is not None:
        c = case
        b, _, h, d = c["q"].shape
        flat = lambda t: None if t is None else t.reshape(b, -1)
        emu_out, emu_lse = orc.emulate_fp8_attention_dual(
            c["q"].view(b, h, d), c["packed"].cpu(), flat(c["indices"]), c["sm_scale"], c["topk_length"],
            None if c["extra_packed"] is None else c["extra_packed"].cpu(), flat(c["extra_indices"]),
            c["extra_topk_length"], c["attn_sink"])
        k = H.lse2_to_nat(lse2.cpu()).view(b, h)
        k = torch.where(k > 1e30, torch.full_like(k, float("inf")), k)
        H.check_against_emulated(out.cpu().view(b, h, 512), k, emu_out, _expected_lse(emu_lse, sink),
                                 ref_out.view(b, h, 512), _expected_lse(ref_lse.view(b, h), sink))
        return
    if impl == FP32:
        H.compare_out(out.cpu(), ref_out, H.SCALAR_ABS, H.SCALAR_REL)
    else:
        H.compare_out(out.cpu(), ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)
    k = H.lse2_to_nat(lse2.cpu())
    r = _expected_lse(ref_lse, sink)
    k = torch.where(k > 1e30, torch.full_like(k, float("inf")), k)
    assert torch.equal(torch.isinf(k), torch.isinf(r)) and torch.equal(torch.sign(k[torch.isinf(k)]), torch.sign(r[torch.isinf(r)]))
    fin = ~torch.isinf(r)
    if fin.any():
        assert float((k - r)[fin].abs().max()) <= (H.SCALAR_LSE if impl == FP32 else H.TC_LSE)


def _m1_case(seed, b, h, topk, extra_topk=0, lengths=False, extra_lengths=False, sink=False, block=64, nblk=64,
             std=0.1, layout="model1"):
    g = torch.Generator().manual_seed(seed)
    d = 512 if layout == "model1" else 576
    quant, dequant = (orc.quantize_kv_model1, orc.dequantize_kv_model1) if layout == "model1" else \
                     (orc.quantize_kv_v32, orc.dequantize_kv_v32)
    c = {"sm_scale": d ** -0.5}
    kv = (torch.randn(nblk, block, 1, d, generator=g) * std).clamp(-10 * std, 10 * std).to(torch.bfloat16)
    c["packed"] = quant(kv)
    c["deq"] = dequant(c["packed"])
    c["q"] = (torch.randn(b, 1, h, d, generator=g) * std).to(torch.bfloat16)
    c["indices"] = torch.randint(0, nblk * block, (b, 1, topk), generator=g, dtype=torch.int32)
    c["indices"][:, :, -10:] = -1
    c["topk_length"] = torch.randint(0, topk + 1, (b,), generator=g, dtype=torch.int32) if lengths else None
    c["extra_packed"] = c["extra_deq"] = c["extra_indices"] = c["extra_topk_length"] = c["attn_sink"] = None
    if extra_topk:
        enb = max(4, (extra_topk * 2 + block - 1) // block)
        ekv = (torch.randn(enb, block, 1, d, generator=g) * std).to(torch.bfloat16)
        c["extra_packed"] = quant(ekv)
        c["extra_deq"] = dequant(c["extra_packed"])
        c["extra_indices"] = torch.randint(0, enb * block, (b, 1, extra_topk), generator=g, dtype=torch.int32)
        if extra_lengths:
            c["extra_topk_length"] = torch.randint(0, extra_topk + 1, (b,), generator=g, dtype=torch.int32)
    if sink:
        s = torch.randn(h, generator=g) * 2.0
        m = torch.randn(h, generator=g)
        s[m > 1.0], s[m < -1.0] = float("inf"), float("-inf")
        c["attn_sink"] = s
    return c


def _oracle(c):
    return orc.ref_sparse_attn_dual(c["q"], c["deq"], c["indices"], c["sm_scale"], 512, c["topk_length"],
                                    c["extra_deq"], c["extra_indices"], c["extra_topk_length"], c["attn_sink"])


def _decode(c, num_sm_parts=None, impl=FP32):
    from sparse_mla_sm120_b200 import flash_ops
    from sparse_mla_sm120_b200._runtime import check_status
    b, _, h, d = c["q"].shape
    etopk = 0 if c["extra_indices"] is None else c["extra_indices"].shape[-1]
    out, lse = flash_ops.sparse_mla_decode_fwd(
        _dev(c["q"]).view(b, h, d), _dev(c["packed"]), _dev(c["indices"]).view(b, -1), c["sm_scale"], 512,
        attn_sink=_dev(c["attn_sink"]), extra_k_cache=_dev(c["extra_packed"]),
        extra_indices=None if etopk == 0 else _dev(c["extra_indices"]).view(b, -1), topk_length=_dev(c["topk_length"]),
        extra_topk_length=_dev(c["extra_topk_length"]), extra_topk=etopk, num_sm_parts=num_sm_parts, impl=impl)
    torch.cuda.synchronize()
    check_status(torch.device(DEV))
    return out.view(b, 1, h, 512), lse.view(b, 1, h)


# ------------------------------------------------------------------ fixtures of the reference's helpers
@pytest.mark.parametrize("name", M1_CASES)
@pytest.mark.parametrize("parts", [None, 3, 40])
def test_model1_golden_decode(golden_dir, name, parts, impl):
    c = load_m1_case(golden_dir, name)
    c["deq"] = c["extra_deq"] = None
    out, lse = _decode(c, num_sm_parts=parts, impl=impl)
    _compare(out, lse, c["out"], c["lse"], c["attn_sink"], impl)


@pytest.mark.parametrize("name", M1_CASES)
def test_model1_golden_flashmla_interface(golden_dir, name, impl):
    from sparse_mla_sm120_b200 import interface
    c = load_m1_case(golden_dir, name)
    meta, _ = interface.get_mla_metadata()
    for _ in range(2):   # the second call reuses the schedule
        out, lse = interface.flash_mla_with_kvcache(
            _dev(c["q"]), _dev(c["packed"]), None, None, 512, meta, None, c["sm_scale"], False, True,
            indices=_dev(c["indices"]), attn_sink=_dev(c["attn_sink"]), extra_k_cache=_dev(c["extra_packed"]),
            extra_indices_in_kvcache=_dev(c["extra_indices"]), topk_length=_dev(c["topk_length"]),
            extra_topk_length=_dev(c["extra_topk_length"]), impl=impl)
        torch.cuda.synchronize()
        _compare(out, lse.permute(0, 2, 1), c["out"], c["lse"], c["attn_sink"], impl)


# ------------------------------------------------------------------ the reference's V4 grid, seeded
@pytest.mark.parametrize("h,topk,b", [(64, 512, 1), (64, 512, 4), (64, 512, 8), (128, 1024, 1), (128, 1024, 4),
                                      (8, 512, 1), (8, 512, 4)])
def test_model1_topk_length(h, topk, b, impl):
    c = _m1_case(42, b, h, topk, lengths=True)
    out, lse = _decode(c, impl=impl)
    _compare(out, lse, *_oracle(c), impl=impl, case=c)


def test_model1_all_lengths_zero(impl):
    c = _m1_case(999, 4, 64, 512, lengths=True)
    c["topk_length"].zero_()
    out, lse = _decode(c, impl=impl)
    assert not out.any()
    assert bool((lse < -1e29).all())


@pytest.mark.parametrize("h,topk,extra,b", [(64, 512, 64, 1), (64, 512, 64, 4), (64, 512, 128, 4), (128, 1024, 128, 1),
                                            (128, 1024, 128, 4), (8, 512, 64, 1)])
@pytest.mark.parametrize("extra_lengths", [False, True])
def test_model1_extra_cache(h, topk, extra, b, extra_lengths, impl):
    c = _m1_case(42, b, h, topk, extra_topk=extra, extra_lengths=extra_lengths)
    for parts in (None, 5):
        out, lse = _decode(c, num_sm_parts=parts, impl=impl)
        _compare(out, lse, *_oracle(c), impl=impl)


@pytest.mark.parametrize("h,topk,b", [(64, 512, 4), (128, 1024, 2), (8, 512, 4)])
def test_model1_sink_with_infinities(h, topk, b, impl):
    c = _m1_case(42, b, h, topk, sink=True)
    ref_out, ref_lse = _oracle(c)
    for parts in (None, 7):
        out, lse = _decode(c, num_sm_parts=parts, impl=impl)
        _compare(out, lse, ref_out, ref_lse, c["attn_sink"], impl)


def test_model1_everything_at_once(impl):
    c = _m1_case(7, 5, 64, 300, extra_topk=100, lengths=True, extra_lengths=True, sink=True, block=32, nblk=40, std=0.5)
    ref_out, ref_lse = _oracle(c)
    for parts in (None, 1, 9):
        out, lse = _decode(c, num_sm_parts=parts, impl=impl)
        _compare(out, lse, ref_out, ref_lse, c["attn_sink"], impl, case=c)


def test_v32_extra_cache(impl):
    """The second cache with the 656-byte layout."""
    c = _m1_case(11, 3, 16, 256, extra_topk=96, lengths=True, extra_lengths=True, layout="v32", nblk=16)
    for parts in (None, 4):
        out, lse = _decode(c, num_sm_parts=parts, impl=impl)
        _compare(out, lse, *_oracle(c), impl=impl, case=c)


def test_model1_padded_page_stride(impl):
    """Pages further apart than block x 584 bytes (flash_mla_sm120/ops.py:23-45)."""
    c = _m1_case(3, 2, 16, 128, nblk=8)
    nb, bs = c["packed"].shape[:2]
    wide = torch.zeros(nb, bs * 584 + 64, dtype=torch.uint8)
    wide[:, :bs * 584] = c["packed"].reshape(nb, -1)
    ref_out, ref_lse = _oracle(c)
    view = _dev(wide)[:, :bs * 584].view(nb, bs, 1, 584)
    assert view.stride(0) == bs * 584 + 64
    c["packed"] = view
    out, lse = _decode(c, impl=impl)
    _compare(out, lse, ref_out, ref_lse, impl=impl)


# ------------------------------------------------------------------ prefill
@pytest.mark.parametrize("h,tokens,topk,extra", [(128, 65, 512, 0), (64, 70, 256, 64), (16, 33, 128, 128)])
def test_model1_prefill(h, tokens, topk, extra, impl):
    from sparse_mla_sm120_b200 import flash_ops, interface
    c = _m1_case(21, tokens, h, topk, extra_topk=extra, lengths=True, sink=True, nblk=32)
    ref_out, ref_lse = _oracle(c)
    q = _dev(c["q"]).view(tokens, h, 512)
    eidx = None if not extra else _dev(c["extra_indices"]).view(tokens, -1)
    out, mx, lse = flash_ops.sparse_mla_prefill_fwd(
        q, _dev(c["packed"]), _dev(c["indices"]).view(tokens, -1), c["sm_scale"], 512, attn_sink=_dev(c["attn_sink"]),
        topk_length=_dev(c["topk_length"]), extra_k_cache=_dev(c["extra_packed"]), extra_indices=eidx, extra_topk=extra,
        impl=impl)
    torch.cuda.synchronize()
    _compare(out.view(tokens, 1, h, 512), lse.view(tokens, 1, h), ref_out, ref_lse, c["attn_sink"], impl, case=c)
    # max_logits: the largest scaled logit of a row in base 2 (prefill_kernel.cuh epilogue), -1e30 for an empty row
    deq = c["deq"].reshape(-1, 512).float()
    out2, mx2, lse2 = interface.flash_mla_sparse_fwd(
        q, _dev(c["packed"]), _dev(c["indices"]), c["sm_scale"], 512, attn_sink=_dev(c["attn_sink"]),
        topk_length=_dev(c["topk_length"]), extra_k_cache=_dev(c["extra_packed"]),
        extra_indices_in_kvcache=eidx)
    torch.cuda.synchronize()
    if impl == FP32:   # the FlashMLA-shaped wrapper runs the default kernel, which for this layout is the fp32 one
        assert torch.equal(out2, out) and torch.equal(lse2, lse) and torch.equal(mx2, mx)
    t = 0
    idx = c["indices"][t, 0]
    valid = (idx >= 0) & (torch.arange(topk) < int(c["topk_length"][t]))
    logits = (c["q"][t, 0].float() @ deq[idx.clamp(min=0).long()].T) * c["sm_scale"] * math.log2(math.e)
    logits[:, ~valid] = -1e30
    best = logits.max(dim=-1).values
    if extra:
        edeq = c["extra_deq"].reshape(-1, 512).float()
        eidx0 = c["extra_indices"][t, 0]
        el = (c["q"][t, 0].float() @ edeq[eidx0.clamp(min=0).long()].T) * c["sm_scale"] * math.log2(math.e)
        el[:, eidx0 < 0] = -1e30
        best = torch.maximum(best, el.max(dim=-1).values)
    tol = 1e-4 if impl == FP32 else 2e-2     # the tensor-core kernel's logits carry the e4m3 rounding of q
    assert torch.allclose(mx[t].cpu(), best, rtol=tol, atol=tol)


# ------------------------------------------------------------------ the raw entry points of the extension module
def test_model1_raw_entry_points(impl):
    """The call sequence of tests/test_v4_features.py:170-207 of the reference, on its argument order."""
    from flash_mla_sm120.cuda import get_decode_metadata, sparse_mla_combine_v2_fwd, sparse_mla_splitkv_v2_fwd
    b, h, topk, extra = 4, 64, 512, 128
    c = _m1_case(42, b, h, topk, extra_topk=extra, lengths=True, extra_lengths=True, sink=True)
    ref_out, ref_lse = _oracle(c)
    parts = 11
    dev = torch.device(DEV)
    sched = torch.empty(parts * 8, dtype=torch.int32, device=dev)
    nsplits = torch.empty(b + 1, dtype=torch.int32, device=dev)
    tl, etl = _dev(c["topk_length"]), _dev(c["extra_topk_length"])
    get_decode_metadata(b, topk, extra, parts, 5, tl, etl, sched, nsplits)
    o_accum = torch.empty(b + parts, 1, h, 512, dtype=torch.float32, device=dev)
    lse_accum = torch.empty(b + parts, 1, h, dtype=torch.float32, device=dev)
    output = torch.zeros(b, h, 512, dtype=torch.bfloat16, device=dev)
    out_lse = torch.zeros(b, h, dtype=torch.float32, device=dev)
    kv, ekv = _dev(c["packed"]), _dev(c["extra_packed"])
    sink = _dev(c["attn_sink"])
    sparse_mla_splitkv_v2_fwd(_dev(c["q"]).view(b, h, 512), kv, _dev(c["indices"]).view(b, topk), o_accum, lse_accum,
                              output, out_lse, sched, nsplits, c["sm_scale"], topk, kv.stride(-2), kv.shape[-3], parts,
                              sink, ekv, _dev(c["extra_indices"]).view(b, extra), tl, extra, etl, True, impl)
    ns = nsplits.cpu()
    sparse_mla_combine_v2_fwd(o_accum, lse_accum, output, out_lse, nsplits, b,
                              int((ns[1:] - ns[:-1]).max()), sink)
    torch.cuda.synchronize()
    _compare(output.view(b, 1, h, 512), out_lse.view(b, 1, h), ref_out, ref_lse, c["attn_sink"], impl, case=c)


def test_layout_mismatch_is_refused():
    from sparse_mla_sm120_b200 import flash_ops
    c = _m1_case(1, 1, 8, 64, nblk=2)
    q576 = torch.zeros(1, 8, 576, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        flash_ops.sparse_mla_decode_fwd(q576, _dev(c["packed"]), _dev(c["indices"]).view(1, -1), 0.1)
    with pytest.raises(ValueError):   # extra_topk without a cache
        flash_ops.sparse_mla_decode_fwd(_dev(c["q"]).view(1, 8, 512), _dev(c["packed"]), _dev(c["indices"]).view(1, -1),
                                        0.1, extra_topk=64)


def test_unaligned_pages_fall_back_to_the_fp32_kernel():
    """The tensor-core kernel's bulk copies need page strides that are multiples of 16 bytes: asked for by name it
    refuses others, left to choose the library runs the fp32 kernel."""
    c = _m1_case(5, 2, 16, 128, nblk=8)
    nb, bs = c["packed"].shape[:2]
    wide = torch.zeros(nb, bs * 584 + 8, dtype=torch.uint8)
    wide[:, :bs * 584] = c["packed"].reshape(nb, -1)
    c["packed"] = _dev(wide)[:, :bs * 584].view(nb, bs, 1, 584)
    with pytest.raises(ValueError, match="aligned"):
        _decode(c, impl=TC)
    # 656-byte rows with a second cache whose pages are 8 bytes further apart than their rows need
    c = _m1_case(6, 2, 16, 128, extra_topk=64, nblk=8, layout="v32")
    ref_out, ref_lse = _oracle(c)
    nb, bs = c["extra_packed"].shape[:2]
    wide = torch.zeros(nb, bs * 656 + 8, dtype=torch.uint8)
    wide[:, :bs * 656] = c["extra_packed"].reshape(nb, -1)
    c["extra_packed"] = _dev(wide)[:, :bs * 656].view(nb, bs, 1, 656)
    out, lse = _decode(c, impl=0)
    _compare(out, lse, ref_out, ref_lse, impl=FP32)
    with pytest.raises(ValueError, match="aligned"):
        _decode(c, impl=TC)


def test_model1_default_kernel_and_its_switch():
    """Left to choose, a MODEL1 call runs the exact fp32 kernel; _runtime.MODEL1_DEFAULT_IMPL (or SMLA_MODEL1_IMPL=tc
    in the environment) makes the tensor-core kernel the default."""
    from sparse_mla_sm120_b200 import _runtime
    c = _m1_case(8, 3, 64, 256, extra_topk=64, nblk=16)
    exact, _ = _decode(c, impl=FP32)
    fast, _ = _decode(c, impl=TC)
    assert not torch.equal(exact, fast)
    assert _runtime.MODEL1_DEFAULT_IMPL == FP32
    auto, _ = _decode(c, impl=0)
    assert torch.equal(auto, exact)
    _runtime.MODEL1_DEFAULT_IMPL = TC
    try:
        auto, _ = _decode(c, impl=0)
    finally:
        _runtime.MODEL1_DEFAULT_IMPL = FP32
    assert torch.equal(auto, fast)
