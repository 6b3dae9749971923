"""Generate the golden fixtures in this folder from the reference's own test helpers.

Run once where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference [v32|model1|all]

The reference's test modules import its CUDA extension at module import; that import is
satisfied with empty stub modules because only the pure-PyTorch helpers are called
(quantize_kv_v32, dequantize_kv_v32, quantize_kv_model1, dequantize_kv_model1 and
ref_sparse_attn_decode from tests/test_decode.py, combine_v2_ref from tests/test_combine.py,
ref_v4_decode from tests/test_v4_features.py).  bf16 tensors are stored as their uint16 bit
patterns so that the .npz files need nothing but numpy to read.
"""
import sys
import types

import numpy as np
import torch


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.contiguous().numpy()


def _stub_extension(ref_root: str) -> None:
    for name in ("flash_mla_sm120", "flash_mla_sm120.cuda"):
        sys.modules[name] = types.ModuleType(name)
    sys.modules["flash_mla_sm120"].cuda = sys.modules["flash_mla_sm120.cuda"]
    for fn in ("get_decode_metadata", "sparse_mla_splitkv_v2_fwd", "sparse_mla_combine_v2_fwd",
               "sparse_mla_prefill_fwd"):
        setattr(sys.modules["flash_mla_sm120.cuda"], fn, None)
    sys.path.insert(0, ref_root + "/tests")


def main_model1(ref_root: str, out_dir: str) -> None:
    """The 584-byte footer layout and attention over it, with the second cache, lengths and sink."""
    _stub_extension(ref_root)
    import test_decode as ref_dec
    import test_v4_features as ref_v4

    torch.manual_seed(7)
    kv = (torch.randn(3, 64, 1, 512, dtype=torch.bfloat16) * torch.tensor([0.1, 1.0, 40.0]).view(3, 1, 1, 1).bfloat16())
    kv[0, 0] = 0  # an all-zero row exercises the 1e-4 amax floor
    packed = ref_dec.quantize_kv_model1(kv)
    deq = ref_dec.dequantize_kv_model1(packed)
    np.savez_compressed(out_dir + "/kv_format_model1.npz", kv_bf16=_bits(kv), packed=packed.numpy(),
                        dequant_bf16=_bits(deq))

    cases = {
        # name: (b, h, topk, extra_topk, lengths?, sink?, block, num_blocks)
        "attn_m1_h16": (2, 16, 128, 0, False, False, 64, 6),
        "attn_m1_h64_extra": (3, 64, 192, 96, True, True, 64, 6),
        "attn_m1_h8_block16": (2, 8, 100, 40, True, False, 16, 20),
    }
    for name, (b, h, topk, etopk, lengths, sink, block, nblk) in cases.items():
        torch.manual_seed(321)
        kv = (torch.randn(nblk, block, 1, 512, dtype=torch.bfloat16) / 2).clamp(-3, 3)
        packed = ref_dec.quantize_kv_model1(kv)
        deq = ref_dec.dequantize_kv_model1(packed)
        q = (torch.randn(b, 1, h, 512, dtype=torch.bfloat16) / 2)
        idx = torch.randint(0, nblk * block, (b, 1, topk), dtype=torch.int32)
        idx[:, :, -10:] = -1
        rec = dict(packed=packed.numpy(), q_bf16=_bits(q), indices=idx.numpy())
        tl = etl = epacked = edeq = eidx = attn_sink = None
        if lengths:
            tl = torch.randint(0, topk + 1, (b,), dtype=torch.int32)
            tl[0] = 0                                  # a request whose main cache contributes nothing
            rec["topk_length"] = tl.numpy()
        if etopk:
            ekv = (torch.randn(4, block, 1, 512, dtype=torch.bfloat16) / 2).clamp(-3, 3)
            epacked = ref_dec.quantize_kv_model1(ekv)
            edeq = ref_dec.dequantize_kv_model1(epacked)
            eidx = torch.randint(0, 4 * block, (b, 1, etopk), dtype=torch.int32)
            eidx[:, :, ::7] = -1
            rec["extra_packed"], rec["extra_indices"] = epacked.numpy(), eidx.numpy()
            if lengths:
                etl = torch.randint(1, etopk + 1, (b,), dtype=torch.int32)
                rec["extra_topk_length"] = etl.numpy()
        if sink:
            attn_sink = torch.randn(h) * 2.0
            attn_sink[3], attn_sink[5] = float("inf"), float("-inf")
            rec["attn_sink"] = attn_sink.numpy()
        sm_scale = 512 ** -0.5
        out, lse = ref_v4.ref_v4_decode(q, deq, idx, sm_scale, 512, topk_length=tl, extra_kv_dequant=edeq,
                                        extra_indices=eidx, extra_topk_length=etl, attn_sink=attn_sink)
        np.savez_compressed(out_dir + f"/{name}.npz", sm_scale=np.float32(sm_scale), out_bf16=_bits(out),
                            lse=lse.numpy(), **rec)
    print("MODEL1 golden fixtures written to", out_dir)


def main(ref_root: str, out_dir: str) -> None:
    _stub_extension(ref_root)
    import test_decode as ref_dec
    import test_combine as ref_comb

    # ---- KV row format -------------------------------------------------------------
    torch.manual_seed(42)
    kv = (torch.randn(4, 64, 1, 576, dtype=torch.bfloat16) * torch.tensor(
        [0.1, 1.0, 7.0, 300.0]).view(4, 1, 1, 1).bfloat16())
    kv[0, 0] = 0  # an all-zero row exercises the 1e-4 amax floor
    packed = ref_dec.quantize_kv_v32(kv)
    deq = ref_dec.dequantize_kv_v32(packed)
    np.savez_compressed(out_dir + "/kv_format.npz", kv_bf16=_bits(kv), packed=packed.numpy(),
                        dequant_bf16=_bits(deq))

    # ---- attention: small decode-like cases -----------------------------------------
    cases = {
        # name: (b, s_q, h, topk, num_blocks, data scale, q scale)
        "attn_h16": (2, 1, 16, 128, 8, 0.1, 0.1),
        "attn_h128": (1, 2, 128, 192, 8, 1.0, 0.5),
        "attn_h64_lonely": (3, 1, 64, 64, 4, 1.0, 0.5),
    }
    for name, (b, s_q, h, topk, nblk, ks, qs) in cases.items():
        torch.manual_seed(123)
        kv = (torch.randn(nblk, 64, 1, 576, dtype=torch.bfloat16) * ks).clamp(-4, 4)
        packed = ref_dec.quantize_kv_v32(kv)
        deq = ref_dec.dequantize_kv_v32(packed)
        q = (torch.randn(b, s_q, h, 576, dtype=torch.bfloat16) * qs)
        idx = torch.stack([torch.randperm(nblk * 64)[:topk] for _ in range(b * s_q)]).view(b, s_q, topk).int()
        idx[:, :, -(topk // 10):] = -1
        if name.endswith("lonely"):
            idx[1] = -1                      # a request with no valid entry at all
            idx[2, :, ::2] = -1              # interleaved invalid entries
        sm_scale = 576 ** -0.5
        out, lse = ref_dec.ref_sparse_attn_decode(q, deq, idx, sm_scale, 512)
        np.savez_compressed(out_dir + f"/{name}.npz", packed=packed.numpy(), q_bf16=_bits(q),
                            indices=idx.numpy(), sm_scale=np.float32(sm_scale),
                            out_bf16=_bits(out), lse=lse.numpy())

    # ---- combine ---------------------------------------------------------------------
    torch.manual_seed(42)
    splits = [2, 5, 1, 8, 3]
    prefix = np.concatenate([[0], np.cumsum(splits)]).astype(np.int32)
    total, h = int(prefix[-1]), 16
    o_accum = torch.randn(total, 1, h, 512) * 0.1
    lse_accum = torch.randn(total, 1, h) * 3.0
    lse_accum[2, 0, :4] = 100.0            # one dominant split
    lse_accum[7:15, 0, 5] = -1e30          # a head whose every split of request 3 is empty
    out, lse = ref_comb.combine_v2_ref(o_accum, lse_accum, torch.from_numpy(prefix), len(splits), h, 512)
    np.savez_compressed(out_dir + "/combine.npz", o_accum=o_accum.numpy(), lse_accum=lse_accum.numpy(),
                        num_splits=prefix, out_bf16=_bits(out), lse=lse.numpy())
    print("golden fixtures written to", out_dir)


if __name__ == "__main__":
    import os
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference [v32|model1|all]")
    which = sys.argv[2] if len(sys.argv) > 2 else "all"
    here = os.path.dirname(os.path.abspath(__file__))
    if which in ("v32", "all"):
        main(sys.argv[1], here)
    if which in ("model1", "all"):
        main_model1(sys.argv[1], here)
