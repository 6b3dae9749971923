"""Generate the golden fixtures in this folder from the reference's own test helpers.

Run once where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

The reference's test modules import its CUDA extension at module import; that import is
satisfied with empty stub modules because only the pure-PyTorch helpers are called
(quantize_kv_v32, dequantize_kv_v32, ref_sparse_attn_decode from tests/test_decode.py and
combine_v2_ref from tests/test_combine.py).  bf16 tensors are stored as their uint16 bit
patterns so that the .npz files need nothing but numpy to read.
"""
import sys
import types

import numpy as np
import torch


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.contiguous().numpy()


def main(ref_root: str, out_dir: str) -> None:
    for name in ("flash_mla_sm120", "flash_mla_sm120.cuda"):
        sys.modules[name] = types.ModuleType(name)
    sys.modules["flash_mla_sm120"].cuda = sys.modules["flash_mla_sm120.cuda"]
    sys.path.insert(0, ref_root + "/tests")
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
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1], os.path.dirname(os.path.abspath(__file__)))
