"""The CPU oracle against the fixtures that the reference's own helpers produced
(tests/golden/make_golden.py).  These pin the oracle; no GPU involved."""
import numpy as np
import torch

from helpers import bf16_from_bits, orc


def _load(golden_dir, name):
    return np.load(f"{golden_dir}/{name}.npz")


def test_kv_format_roundtrip(golden_dir):
    g = _load(golden_dir, "kv_format")
    kv = bf16_from_bits(g["kv_bf16"])
    packed = orc.quantize_kv_v32(kv)
    assert np.array_equal(packed.numpy(), g["packed"]), "packed bytes differ from the reference writer"
    deq = orc.dequantize_kv_v32(torch.from_numpy(g["packed"]))
    assert np.array_equal(deq.view(torch.uint16).numpy(), g["dequant_bf16"]), "dequantised bf16 differs"
    # every stored scale is a power of two (the kernels rely on it)
    scales = torch.from_numpy(g["packed"]).reshape(-1, 656)[:, 512:528].contiguous().view(torch.float32)
    m, _ = torch.frexp(scales)
    assert torch.all(m == 0.5)


def test_attention_matches_reference(golden_dir):
    for name in ("attn_h16", "attn_h128", "attn_h64_lonely"):
        g = _load(golden_dir, name)
        packed = torch.from_numpy(g["packed"])
        q = bf16_from_bits(g["q_bf16"])
        idx = torch.from_numpy(g["indices"])
        out, lse = orc.ref_sparse_attn(q, orc.dequantize_kv_v32(packed), idx, float(g["sm_scale"]), 512)
        ref_out = bf16_from_bits(g["out_bf16"])
        assert torch.equal(out.view(torch.uint16), ref_out.view(torch.uint16)), name
        ref_lse = torch.from_numpy(g["lse"])
        assert torch.equal(torch.isinf(lse), torch.isinf(ref_lse)), name
        fin = ~torch.isinf(ref_lse)
        assert torch.allclose(lse[fin], ref_lse[fin], rtol=0, atol=1e-6), name
    # the lonely request: output exactly zero, LSE -inf
    g = _load(golden_dir, "attn_h64_lonely")
    assert not bf16_from_bits(g["out_bf16"])[1].any()
    assert np.all(np.isneginf(g["lse"][1]))


def test_combine_matches_reference(golden_dir):
    g = _load(golden_dir, "combine")
    out, lse = orc.combine_ref(torch.from_numpy(g["o_accum"]), torch.from_numpy(g["lse_accum"]),
                               g["num_splits"].tolist(), len(g["num_splits"]) - 1)
    assert torch.equal(out.view(torch.uint16), bf16_from_bits(g["out_bf16"]).view(torch.uint16))
    assert torch.equal(lse, torch.from_numpy(g["lse"]))


def test_topk_length_masks_tail():
    from helpers import make_case
    c = make_case(3, 2, 8, 128, 4, invalid_tail=0.0)
    tl = torch.tensor([40, 128], dtype=torch.int32)
    deq = orc.dequantize_kv_v32(c["packed"])
    out, lse = orc.ref_sparse_attn(c["q"].unsqueeze(1), deq, c["indices"].unsqueeze(1), c["sm_scale"], 512, tl)
    idx2 = c["indices"].clone()
    idx2[0, 40:] = -1
    out2, lse2 = orc.ref_sparse_attn(c["q"].unsqueeze(1), deq, idx2.unsqueeze(1), c["sm_scale"], 512)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)


def test_fp8_emulation_distance():
    """The numbers the tensor-core tolerances of helpers.py are derived from: distance of the emulated FP8-class
    numerics to the fp32 oracle on reference-grid and benchmark-like data."""
    import helpers as H
    case = H.make_case(2, 2, 128, 1024, 32, kv_std=0.1, q_std=0.1, clamp=1.0)
    ref_out, ref_lse = H.oracle_attn(case)
    emu_out, emu_lse = orc.emulate_fp8_attention(case["q"], case["packed"], case["indices"], case["sm_scale"])
    assert float((emu_out.float() - ref_out.float()).abs().max()) < 1e-3          # the reference's bar on its own data
    case = H.make_case(4, 3, 64, 512, 32, kv_std=1.0, q_std=0.5)
    ref_out, ref_lse = H.oracle_attn(case)
    emu_out, emu_lse = orc.emulate_fp8_attention(case["q"], case["packed"], case["indices"], case["sm_scale"])
    H.compare_out(emu_out, ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)                 # the emulation sits inside the kernel bounds
    fin = torch.isfinite(ref_lse)
    assert float((emu_lse[fin] - ref_lse[fin]).abs().max()) < H.TC_LSE
    d = (emu_out.float() - ref_out.float()).abs()
    rms = float(ref_out.float().pow(2).mean().sqrt())
    excess = float((d - (H.TC_ABS + H.TC_REL * torch.maximum(emu_out.float().abs(), ref_out.float().abs()))).max()) / rms
    assert 0.03 < excess < H.TC_NOISE / 1.3, excess                               # TC_NOISE keeps >= 1.3 x margin over it


def test_fp8_emulation_of_both_layouts_and_two_caches(golden_dir):
    """emulate_fp8_attention_dual: on V32 inputs without a second cache it is emulate_fp8_attention; on the MODEL1
    fixtures (second cache, lengths, sink) it stays inside the fixed FP8-class bounds around the reference's results."""
    import helpers as H
    case = H.make_case(3, 4, 16, 256, 8)
    a = orc.emulate_fp8_attention(case["q"], case["packed"], case["indices"], case["sm_scale"])
    b = orc.emulate_fp8_attention_dual(case["q"], case["packed"], case["indices"], case["sm_scale"])
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    for name in M1_CASES:
        c = load_m1_case(golden_dir, name)
        bq, _, h, d = c["q"].shape
        flat = lambda t: None if t is None else t.reshape(bq, -1)  # noqa: E731
        out, lse = orc.emulate_fp8_attention_dual(c["q"].view(bq, h, d), c["packed"], flat(c["indices"]), c["sm_scale"],
                                                  c["topk_length"], c["extra_packed"], flat(c["extra_indices"]),
                                                  c["extra_topk_length"], c["attn_sink"])
        H.compare_out(out, c["out"].view(bq, h, 512), H.TC_ABS, H.TC_REL, H.TC_COS)
        ref = c["lse"].view(bq, h)
        fin = torch.isfinite(ref)
        assert torch.equal(torch.isfinite(lse), fin)
        assert float((lse[fin] - ref[fin]).abs().max()) < H.TC_LSE


M1_CASES = ("attn_m1_h16", "attn_m1_h64_extra", "attn_m1_h8_block16")


def load_m1_case(golden_dir, name):
    """A MODEL1 fixture as CPU tensors (absent arrays -> None)."""
    g = _load(golden_dir, name)
    t = lambda k: torch.from_numpy(g[k]) if k in g else None  # noqa: E731
    return {"packed": t("packed"), "q": bf16_from_bits(g["q_bf16"]), "indices": t("indices"),
            "topk_length": t("topk_length"), "extra_packed": t("extra_packed"), "extra_indices": t("extra_indices"),
            "extra_topk_length": t("extra_topk_length"), "attn_sink": t("attn_sink"),
            "sm_scale": float(g["sm_scale"]), "out": bf16_from_bits(g["out_bf16"]), "lse": t("lse")}


def test_model1_format_roundtrip(golden_dir):
    g = _load(golden_dir, "kv_format_model1")
    kv = bf16_from_bits(g["kv_bf16"])
    assert np.array_equal(orc.quantize_kv_model1(kv).numpy(), g["packed"]), "footer-ordered bytes differ from the reference writer"
    deq = orc.dequantize_kv_model1(torch.from_numpy(g["packed"]))
    assert np.array_equal(deq.view(torch.uint16).numpy(), g["dequant_bf16"]), "dequantised bf16 differs"
    # the footer of a page starts after block x 576 data bytes and its pad bytes are zero
    page = torch.from_numpy(g["packed"]).reshape(3, 64 * 584)
    assert not page[:, 64 * 576:].reshape(3, 64, 8)[..., 7].any()


def test_model1_attention_matches_reference(golden_dir):
    for name in M1_CASES:
        c = load_m1_case(golden_dir, name)
        edeq = None if c["extra_packed"] is None else orc.dequantize_kv_model1(c["extra_packed"])
        out, lse = orc.ref_sparse_attn_dual(c["q"], orc.dequantize_kv_model1(c["packed"]), c["indices"], c["sm_scale"],
                                            512, c["topk_length"], edeq, c["extra_indices"], c["extra_topk_length"],
                                            c["attn_sink"])
        assert torch.equal(out.view(torch.uint16), c["out"].view(torch.uint16)), name
        assert torch.equal(lse, c["lse"]), name


def test_dual_attention_without_extras_is_the_v32_oracle():
    """ref_sparse_attn_dual restricted to one cache, no lengths and no sink is ref_sparse_attn."""
    from helpers import make_case
    c = make_case(5, 2, 8, 128, 4)
    deq = orc.dequantize_kv_v32(c["packed"])
    a = orc.ref_sparse_attn(c["q"].unsqueeze(1), deq, c["indices"].unsqueeze(1), c["sm_scale"], 512)
    b = orc.ref_sparse_attn_dual(c["q"].unsqueeze(1), deq, c["indices"].unsqueeze(1), c["sm_scale"], 512)
    assert torch.equal(a[0].view(torch.uint16), b[0].view(torch.uint16)) and torch.equal(a[1], b[1])
