"""Parity of the CUDA attention kernels (through the C-ABI) with the CPU oracle.

Each case builds seeded inputs on the CPU, runs the oracle there and the kernels on cuda:0.
``impl`` 1 is the exact fp32 kernel, 2 the tcgen05 kernel (FP8 class; tolerances in helpers.py),
3 the tcgen05 kernel that shares the score work inside a two-CTA cluster (same class).
"""
import numpy as np
import pytest
import torch

import helpers as H
from helpers import bf16_from_bits, make_case, oracle_attn, orc

pytestmark = pytest.mark.gpu

SCALAR, TC = 1, 2


def _tols(impl, prefill=False):
    if impl == SCALAR:
        return H.SCALAR_ABS, H.SCALAR_REL, None, H.SCALAR_LSE
    if prefill:
        return H.TC_PREFILL_ABS, H.TC_PREFILL_REL, H.TC_COS, H.TC_LSE
    return H.TC_ABS, H.TC_REL, H.TC_COS, H.TC_LSE


def _decode(case, impl, num_sm_parts=None, topk_length=None, attn_sink=None):
    from sparse_mla_sm120_b200 import flash_ops
    from sparse_mla_sm120_b200._runtime import check_status
    dev = torch.device("cuda:0")
    tl = None if topk_length is None else topk_length.to(dev)
    sink = None if attn_sink is None else attn_sink.to(dev)
    out, lse = flash_ops.sparse_mla_decode_fwd(case["q"].to(dev), case["packed"].to(dev), case["indices"].to(dev),
                                               case["sm_scale"], 512, attn_sink=sink, topk_length=tl, impl=impl,
                                               num_sm_parts=num_sm_parts)
    torch.cuda.synchronize()
    check_status(dev)
    return out.cpu(), lse.cpu()


def _prefill(case, impl, topk_length=None, attn_sink=None):
    from sparse_mla_sm120_b200 import flash_ops
    from sparse_mla_sm120_b200._runtime import check_status
    dev = torch.device("cuda:0")
    tl = None if topk_length is None else topk_length.to(dev)
    sink = None if attn_sink is None else attn_sink.to(dev)
    out, mx, lse = flash_ops.sparse_mla_prefill_fwd(case["q"].to(dev), case["packed"].to(dev),
                                                    case["indices"].to(dev), case["sm_scale"], 512, attn_sink=sink,
                                                    topk_length=tl, impl=impl)
    torch.cuda.synchronize()
    check_status(dev)
    return out.cpu(), mx.cpu(), lse.cpu()


def _check(out, lse2, ref_out, ref_lse, impl, prefill=False):
    a, r, c, l = _tols(impl, prefill)
    H.compare_out(out, ref_out, a, r, c)
    H.compare_lse(lse2, ref_lse, l)


def _check_hard(out, lse2, ref_out, ref_lse, impl, case, topk_length=None):
    """Inputs on which the FP8 roundings cost more than on benchmark-like data: the exact kernel keeps its
    bound, the tensor-core kernels are held to what the emulated numerics cost on the same inputs."""
    if impl == SCALAR:
        _check(out, lse2, ref_out, ref_lse, impl)
    else:
        H.check_against_emulation(out, lse2, case, ref_out, ref_lse, topk_length=topk_length)


# ------------------------------------------------------------------ golden fixtures
@pytest.mark.parametrize("impl", [SCALAR, TC])
@pytest.mark.parametrize("name", ["attn_h16", "attn_h128", "attn_h64_lonely"])
def test_golden_fixtures(golden_dir, name, impl):
    g = np.load(f"{golden_dir}/{name}.npz")
    q = bf16_from_bits(g["q_bf16"])
    b, s_q, h, _ = q.shape
    case = {"packed": torch.from_numpy(g["packed"]), "q": q.reshape(b * s_q, h, 576).contiguous(),
            "indices": torch.from_numpy(g["indices"]).reshape(b * s_q, -1).contiguous(),
            "sm_scale": float(g["sm_scale"])}
    ref_out = bf16_from_bits(g["out_bf16"]).reshape(b * s_q, h, 512)
    ref_lse = torch.from_numpy(g["lse"]).reshape(b * s_q, h)
    for parts in (None, 1, 3):
        out, lse = _decode(case, impl, num_sm_parts=parts)
        _check(out, lse, ref_out, ref_lse, impl)
    out, mx, lse = _prefill(case, impl)
    _check(out, lse, ref_out, ref_lse, impl, prefill=True)
    if name.endswith("lonely"):
        assert not out.view(b, s_q, h, 512)[1].any(), "a request without valid entries must give exact zeros"


# ------------------------------------------------------------------ reference test grid (tests/test_decode.py:223-234)
@pytest.mark.parametrize("impl", [SCALAR, TC])
@pytest.mark.parametrize("num_heads,batch", [(128, 1), (128, 4), (16, 1), (16, 4), (64, 1), (64, 4), (8, 1), (8, 4)])
def test_decode_reference_grid(num_heads, batch, impl):
    """topk 2048, data randn/10 clamped, last 10 indices -1, bound max|dO| < 1e-3 as the reference."""
    case = make_case(42, batch, num_heads, 2048, 64, kv_std=0.1, q_std=0.1, invalid_tail=0.0, clamp=1.0,
                     unique=False)
    case["indices"][:, -10:] = -1
    ref_out, ref_lse = oracle_attn(case)
    out, lse = _decode(case, impl)
    assert float((out.float() - ref_out.float()).abs().max()) < 1e-3
    _check(out, lse, ref_out, ref_lse, impl)


@pytest.mark.parametrize("impl", [SCALAR, TC])
def test_decode_v32_shape_values(impl):
    """Benchmark-like value distribution (kv randn, q randn*0.5), mixed per-tile scales."""
    case = make_case(7, 6, 128, 2048, 96, kv_std=1.0, q_std=0.5, invalid_tail=0.1)
    ref_out, ref_lse = oracle_attn(case)
    for parts in (None, 6, 5):
        out, lse = _decode(case, impl, num_sm_parts=parts)
        _check(out, lse, ref_out, ref_lse, impl)


@pytest.mark.parametrize("impl", [SCALAR, TC])
def test_scale_spread_rows(impl):
    """Rows whose four tiles carry very different scales exercise the re-expression against the
    largest scale."""
    case = make_case(11, 2, 128, 256, 8, q_std=0.06, invalid_tail=0.0)   # small q: the logits stay moderate
    kv = case["kv_bf16"].float()
    kv[..., 128:256] *= 1 / 64.0
    kv[..., 256:384] *= 8.0
    kv[1::3, :, :, 384:512] *= 1e-3
    case["packed"] = orc.quantize_kv_v32(kv.to(torch.bfloat16))
    ref_out, ref_lse = oracle_attn(case)
    out, lse = _decode(case, impl)
    _check_hard(out, lse, ref_out, ref_lse, impl, case)
    if impl != SCALAR:
        # every 128-dim output tile against ITS OWN magnitude (the 8x tile would otherwise hide the 1/64 and
        # 1e-3 tiles): the re-expression against the largest scale must not cost a small tile its precision
        emu_out, _ = orc.emulate_fp8_attention(case["q"], case["packed"], case["indices"], case["sm_scale"])
        for c in range(4):
            sl = slice(128 * c, 128 * c + 128)
            e_k = (out.cpu().float()[..., sl] - ref_out.float()[..., sl]).pow(2).mean().sqrt()
            e_e = (emu_out.float()[..., sl] - ref_out.float()[..., sl]).pow(2).mean().sqrt()
            rms = ref_out.float()[..., sl].pow(2).mean().sqrt()
            assert float(e_k) <= H.EMU_MARGIN * float(e_e) + 2.0 ** -8 * float(rms), (c, float(e_k), float(e_e), float(rms))


@pytest.mark.parametrize("impl", [SCALAR, TC])
def test_peaked_attention_and_rescale(impl):
    """Logits that keep growing along the index list force accumulator rescales; a few dominant
    keys make the distribution peaked.  With logits of +-6 the e4m3 rounding of Q alone moves
    single weights by 10-15 %: the FP8 kernels are held to the emulated numerics on the same inputs."""
    case = make_case(5, 2, 64, 512, 16, kv_std=1.0, q_std=1.5, invalid_tail=0.0)
    deq = orc.dequantize_kv_v32(case["packed"]).reshape(-1, 576).float()
    # order each request's indices by ascending logit of head 0, so the maximum rises to the end
    for t in range(2):
        s = deq[case["indices"][t].long()] @ case["q"][t, 0].float()
        case["indices"][t] = case["indices"][t][torch.argsort(s)]
    ref_out, ref_lse = oracle_attn(case)
    out, lse = _decode(case, impl, num_sm_parts=2)
    _check_hard(out, lse, ref_out, ref_lse, impl, case)


@pytest.mark.parametrize("impl", [SCALAR, TC])
def test_topk_length_and_ragged(impl):
    case = make_case(9, 5, 32, 512, 16, invalid_tail=0.0)
    tl = torch.tensor([512, 100, 0, 64, 333], dtype=torch.int32)
    ref_out, ref_lse = oracle_attn(case, topk_length=tl)
    for parts in (None, 4):
        out, lse = _decode(case, impl, num_sm_parts=parts, topk_length=tl)
        _check(out, lse, ref_out, ref_lse, impl)
    out, mx, lse = _prefill(case, impl, topk_length=tl)
    _check(out, lse, ref_out, ref_lse, impl, prefill=True)
    assert not out[2].any()


@pytest.mark.parametrize("impl", [SCALAR, TC])
def test_minus_one_handling_is_exact(impl):
    """Moving the -1 entries around, or poisoning the row that -1 would be clamped to with NaN,
    must not change a single bit (tests/test_nan_safe.py:13-32 poisons slot 0 the same way)."""
    case = make_case(13, 3, 128, 256, 8, invalid_tail=0.25)
    base_out, base_lse = _decode(case, impl)
    assert torch.isfinite(base_out.float()).all()
    # (a) NaN-poison slot 0, which no valid index uses
    poisoned = dict(case)
    idx = case["indices"].clone()
    idx[idx == 0] = 1
    poisoned["indices"] = idx
    ref_out, ref_lse = _decode(poisoned, impl)
    pk = case["packed"].clone()
    pk.view(-1, 656)[0, :512] = 0x7F
    pk.view(-1, 656)[0, 528:] = torch.tensor([0xC0, 0x7F] * 64, dtype=torch.uint8)
    poisoned["packed"] = pk
    out, lse = _decode(poisoned, impl)
    assert torch.equal(out.view(torch.uint16), ref_out.view(torch.uint16)) and torch.equal(lse, ref_lse)
    # (b) -1 entries inside whole 64-entry blocks at the front instead of the tail
    moved = dict(case)
    idx = case["indices"].clone()
    idx = torch.cat([idx[:, 192:], idx[:, :192]], dim=1).contiguous()   # the 64 invalid entries lead
    moved["indices"] = idx
    out2, lse2 = _decode(moved, impl, num_sm_parts=1)
    o_ref, l_ref = oracle_attn(moved)
    _check(out2, lse2, o_ref, l_ref, impl)


@pytest.mark.parametrize("impl", [SCALAR, TC])
def test_attn_sink(impl):
    case = make_case(21, 4, 64, 512, 16, invalid_tail=0.1)
    case["indices"][3] = -1
    sink = torch.tensor([-float("inf"), 20.0, 0.0, -15.0] * 16, dtype=torch.float32)
    ref_out, ref_lse = oracle_attn(case)
    s_out, s_lse = orc.apply_attn_sink(ref_out, ref_lse, sink)
    for parts in (None, 3):
        out, lse = _decode(case, impl, num_sm_parts=parts, attn_sink=sink)
        a, r, c, l = _tols(impl)
        H.compare_out(out, s_out, a, r, c)
        k = lse.double() * H.LN2
        fin = torch.isfinite(s_lse)
        assert float((k[fin] - s_lse.double()[fin]).abs().max()) <= max(l, 1e-3)
        assert torch.all(k[~fin] < -1e20)


@pytest.mark.parametrize("impl", [SCALAR, TC])
@pytest.mark.parametrize("num_heads,num_tokens", [(128, 65), (64, 65), (16, 100)])
def test_prefill_reference_grid(num_heads, num_tokens, impl):
    """tests/test_prefill.py:56-71: topk 2048, randn/10 data, bound 1e-3; plus max_logits."""
    case = make_case(42, num_tokens, num_heads, 2048, 64, kv_std=0.1, q_std=0.1, invalid_tail=0.0, clamp=1.0,
                     unique=False)
    case["indices"][:, -10:] = -1
    ref_out, ref_lse = oracle_attn(case)
    out, mx, lse = _prefill(case, impl)
    assert float((out.float() - ref_out.float()).abs().max()) < 1e-3
    _check(out, lse, ref_out, ref_lse, impl, prefill=True)
    # max_logits: running maximum of the scaled logits in base 2
    deq = orc.dequantize_kv_v32(case["packed"]).reshape(-1, 576).float()
    t = 0
    valid = case["indices"][t] >= 0
    s = (case["q"][t].float() @ deq[case["indices"][t][valid].long()].T) * case["sm_scale"] * 1.4426950408889634
    assert float((mx[t] - s.max(dim=1).values).abs().max()) < (2e-2 if impl != SCALAR else 1e-4)


def test_out_argument_is_written_in_place():
    from sparse_mla_sm120_b200 import flash_ops
    dev = torch.device("cuda:0")
    case = make_case(2, 3, 16, 128, 4)
    out = torch.zeros(3, 16, 512, dtype=torch.bfloat16, device=dev)
    res, _ = flash_ops.sparse_mla_decode_fwd(case["q"].to(dev), case["packed"].to(dev), case["indices"].to(dev),
                                             case["sm_scale"], out=out, num_sm_parts=3)   # one whole request per partition
    assert res.data_ptr() == out.data_ptr() and out.any()
    out2 = torch.zeros_like(out)
    res2, _, _ = flash_ops.sparse_mla_prefill_fwd(case["q"].to(dev), case["packed"].to(dev),
                                                  case["indices"].to(dev), case["sm_scale"], out=out2)
    assert res2.data_ptr() == out2.data_ptr()
    assert torch.equal(out, out2), "decode and prefill must agree bit for bit on the same inputs"


def test_legacy_surface_and_determinism():
    import sparse_mla_sm120_b200 as smla
    dev = torch.device("cuda:0")
    case = make_case(4, 70, 128, 256, 8)
    q, kv, idx = case["q"].to(dev), case["packed"].view(-1, 1, 656).to(dev), case["indices"].to(dev)
    a = smla.sparse_mla_fwd(q, kv, idx, case["sm_scale"])           # > 64 tokens: prefill
    b = smla.sparse_mla_prefill_fwd(q, kv, idx, case["sm_scale"])
    c = smla.sparse_mla_decode_fwd(q[:8].contiguous(), kv, idx[:8].contiguous(), case["sm_scale"])
    d = smla.sparse_mla_fwd(q[:8].contiguous(), kv, idx[:8].contiguous(), case["sm_scale"])
    assert a.shape == (70, 128, 512) and a.dtype == torch.bfloat16
    assert torch.equal(a, b) and torch.equal(c, d)
    ref_out, _ = oracle_attn(case)
    H.compare_out(a.cpu(), ref_out, H.TC_PREFILL_ABS, H.TC_PREFILL_REL, H.TC_COS)


def test_padded_page_stride():
    """A cache whose pages are padded (page stride > 64*656) is addressed by page."""
    from sparse_mla_sm120_b200 import flash_ops
    dev = torch.device("cuda:0")
    case = make_case(6, 2, 16, 128, 8)
    nb, stride = 8, 64 * 656 + 256
    buf = torch.zeros(nb * stride, dtype=torch.uint8, device=dev)
    kv = torch.as_strided(buf, (nb, 64, 1, 656), (stride, 656, 656, 1))
    kv.copy_(case["packed"].to(dev))
    ref_out, ref_lse = oracle_attn(case)
    out, lse = flash_ops.sparse_mla_decode_fwd(case["q"].to(dev), kv, case["indices"].to(dev), case["sm_scale"])
    H.compare_out(out.cpu(), ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)


@pytest.mark.parametrize("impl", [TC])
def test_many_tokens_per_cta(impl):
    """More query tokens than CTA pairs: without a scheduler every pair walks a run of tokens
    (Q reloaded, accumulator restarted, rings and barrier phases carried over between them)."""
    case = make_case(21, 200, 128, 192, 8, kv_std=1.0, q_std=0.5, invalid_tail=0.05)
    tl = torch.full((200,), 192, dtype=torch.int32)
    tl[::7] = 64          # some tokens with one tile, so that tile ownership flips between tokens
    tl[3::11] = 0         # and some with none
    ref_out, ref_lse = oracle_attn(case, topk_length=tl)
    # 13 M outputs, many of them averages over 64 tokens only
    out, mx, lse = _prefill(case, impl, topk_length=tl)
    _check_hard(out, lse, ref_out, ref_lse, impl, case, topk_length=tl)
    out, lse = _decode(case, impl, num_sm_parts=200, topk_length=tl)     # the unsplit decode path takes the same route
    _check_hard(out, lse, ref_out, ref_lse, impl, case, topk_length=tl)


@pytest.mark.parametrize("impl", [TC])
@pytest.mark.parametrize("magnitude", [0.1, 0.5, 1.0, 2.0, 5.0])
def test_precision_vs_magnitude(impl, magnitude):
    """The reference's magnitude sweep for the 656-byte layout (tests/test_precision_magnitude.py:201-232):
    q and kv are randn x magnitude, 128 heads, top-k 2048; mean |error| / mean |reference| must stay below
    10 %, for decode (2 requests) and prefill (4 tokens)."""
    g = torch.Generator().manual_seed(42)
    kv = (torch.randn(64, 64, 1, 576, generator=g) * magnitude).to(torch.bfloat16)
    packed = orc.quantize_kv_v32(kv)
    q = (torch.randn(4, 128, 576, generator=g) * magnitude).to(torch.bfloat16)
    idx = torch.randint(0, 64 * 64, (4, 2048), generator=g, dtype=torch.int32)
    case = {"packed": packed, "q": q, "indices": idx, "sm_scale": 576 ** -0.5}
    ref_out, _ = oracle_attn(case)
    out_p, _, _ = _prefill(case, impl)
    two = {"packed": packed, "q": q[:2].contiguous(), "indices": idx[:2].contiguous(), "sm_scale": case["sm_scale"]}
    out_d, _ = _decode(two, impl)
    for name, o, r in (("prefill", out_p, ref_out), ("decode", out_d, ref_out[:2])):
        rel = float((o.cpu().float() - r.float()).abs().mean()) / float(r.float().abs().mean())
        assert rel < 0.10, f"{name}: relative error {rel:.3%} at magnitude {magnitude}"


@pytest.mark.parametrize("impl", [SCALAR, TC])
@pytest.mark.parametrize("topk", [1, 100, 257])
def test_topk_not_a_multiple_of_the_block(impl, topk):
    """Index lists of any length: the last block of a list is partly filled."""
    case = make_case(61, 3, 128, topk, 8, invalid_tail=0.0)
    ref_out, ref_lse = oracle_attn(case)
    # a row that averages fewer keys than one block shows Q's e4m3 rounding undamped
    check = (lambda o, l, **kw: _check_hard(o, l, ref_out, ref_lse, impl, case)) if topk < 64 else \
            (lambda o, l, **kw: _check(o, l, ref_out, ref_lse, impl, **kw))
    for parts in (None, 2):
        out, lse = _decode(case, impl, num_sm_parts=parts)
        check(out, lse)
    out, mx, lse = _prefill(case, impl)
    check(out, lse, prefill=True)


# ------------------------------------------------------------------ equal partitions without a scheduler launch
@pytest.mark.parametrize("tokens,heads,topk,k", [(3, 128, 1024, 4), (5, 64, 512, 2), (1, 16, 2048, 8)])
def test_uniform_split_derived_in_the_kernel(tokens, heads, topk, k):
    """Requests of equal length cut into k equal partitions each (smla_decode_uniform: the attention kernel derives the
    schedule, the combine merges k records per request): against the oracle, with a sink, a -1 tail and a request
    whose entries are all -1, and against the same step through the scheduler kernel."""
    import ctypes
    from sparse_mla_sm120_b200 import _lib, flash_ops
    from sparse_mla_sm120_b200._runtime import check_status, kv_geometry, ptr, status_buffer, stream_ptr
    case = make_case(77 + tokens, tokens, heads, topk, 32, invalid_tail=0.2)
    case["indices"][tokens - 1] = -1
    sink = torch.linspace(-1.5, 2.0, heads)
    ref_out, ref_lse = oracle_attn(case)
    ref_out, ref_lse_sink = H.orc.apply_attn_sink(ref_out, ref_lse, sink)
    dev = torch.device("cuda:0")
    q, kv, idx = case["q"].to(dev), case["packed"].to(dev), case["indices"].to(dev)
    pbs, pstride = kv_geometry(kv)
    o_accum = torch.empty(k * tokens, heads, 512, dtype=torch.float32, device=dev)
    lse_accum = torch.empty(k * tokens, heads, dtype=torch.float32, device=dev)
    out = torch.empty(tokens, heads, 512, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(tokens, heads, dtype=torch.float32, device=dev)
    _lib.check(_lib.load().smla_decode_uniform(ptr(q), ptr(kv), ptr(idx), ptr(o_accum), ptr(lse_accum), ptr(out), ptr(lse),
                                               tokens, heads, topk, ctypes.c_float(case["sm_scale"]), pbs, pstride, k,
                                               ptr(sink.to(dev)), TC, ptr(status_buffer(dev)), stream_ptr(dev)))
    torch.cuda.synchronize()
    check_status(dev)
    _check_hard(out.cpu(), lse.cpu(), ref_out, ref_lse_sink, TC, case)
    s_out, s_lse = flash_ops.sparse_mla_decode_fwd(q, kv, idx, case["sm_scale"], attn_sink=sink.to(dev), num_sm_parts=k * tokens)
    torch.cuda.synchronize()
    assert float((s_out.float() - out.float()).abs().max()) <= 2 * H.TC_ABS + H.TC_NOISE * float(ref_out.float().pow(2).mean().sqrt())
    # refused: a partition count that does not divide the blocks, and the fp32 kernel
    lib = _lib.load()
    assert lib.smla_decode_uniform(ptr(q), ptr(kv), ptr(idx), ptr(o_accum), ptr(lse_accum), ptr(out), ptr(lse), tokens, heads,
                                   topk, ctypes.c_float(1.0), pbs, pstride, 3 if (topk // 64) % 3 else 5, None, TC, None,
                                   stream_ptr(dev)) == -2
    assert lib.smla_decode_uniform(ptr(q), ptr(kv), ptr(idx), ptr(o_accum), ptr(lse_accum), ptr(out), ptr(lse), tokens, heads,
                                   topk, ctypes.c_float(1.0), pbs, pstride, k, None, SCALAR, None, stream_ptr(dev)) == -2
