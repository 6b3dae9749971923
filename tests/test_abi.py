"""The C-ABI library: it loads, exports every function include/smla.h declares, and rejects bad
arguments with an error code and a message before touching the device (no GPU needed)."""
import ctypes
import os
import re

import pytest

from helpers import ROOT
from sparse_mla_sm120_b200 import _lib, build


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def _declared():
    text = open(os.path.join(ROOT, "include", "smla.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(smla_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared()
    assert len(names) >= 12
    raw = ctypes.CDLL(build.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/smla.h but not exported"
    assert set(names) == set(_lib.EXPORTS), "python prototypes out of sync with the header"


def test_argument_errors_do_not_launch(lib):
    assert lib.smla_version() >= 100
    rc = lib.smla_decode_splitkv(None, None, None, None, None, None, None, None, None, 1, 128, 2048, 1.0, 64,
                                 64 * 656, 1, None, None, 0, None, None)
    assert rc == -1 and b"null" in lib.smla_last_error()
    fake = 4096  # a non-null, 16-byte aligned address that is never dereferenced on the host
    rc = lib.smla_prefill(fake, fake, fake, fake, fake, None, 1, 129, 2048, 1.0, 64, 64 * 656, None, None, 0,
                          None, None)
    assert rc == -2 and b"num_heads" in lib.smla_last_error()
    rc = lib.smla_prefill(fake + 4, fake, fake, fake, fake, None, 1, 128, 2048, 1.0, 64, 64 * 656, None, None, 0,
                          None, None)
    assert rc == -3
    rc = lib.smla_prefill(fake, fake, fake, fake, fake, None, 1, 128, 2048, 1.0, 64, 64 * 600, None, None, 0,
                          None, None)
    assert rc == -2 and b"stride" in lib.smla_last_error()
    assert lib.smla_combine(fake, fake, fake, fake, fake, 1, 128, 4096, None, None) == -2
    assert lib.smla_sched_meta(0, 2048, 0, 4, 5, None, None, fake, fake, None) == -2
    assert lib.smla_topk(None, None, None, None, 1, 1, 1, 1, None) == -1
    assert lib.smla_workspace_bytes(64, 128, 74) == (64 + 74) * 128 * 513 * 4
    with pytest.raises(ValueError):
        _lib.check(-2)


def test_python_surface_rejects_cpu_tensors_and_mismatched_layouts():
    """There is no CPU path, and q's width must go with the cache layout (576 with 656-byte rows, 512 with the
    584-byte footer layout); all refused before any device work."""
    import torch
    import sparse_mla_sm120_b200 as smla
    q = torch.zeros(1, 128, 576, dtype=torch.bfloat16)
    kv = torch.zeros(4, 64, 1, 656, dtype=torch.uint8)
    kv_m1 = torch.zeros(4, 64, 1, 584, dtype=torch.uint8)
    idx = torch.zeros(1, 64, dtype=torch.int32)
    with pytest.raises(ValueError, match="CUDA"):
        smla.flash_ops.sparse_mla_decode_fwd(q, kv, idx, 1.0)
    with pytest.raises(ValueError, match="CUDA"):
        smla.flash_ops.sparse_mla_decode_fwd(q[..., :512].contiguous(), kv_m1, idx, 1.0)
    with pytest.raises(ValueError, match="does not go with"):
        smla.flash_ops.sparse_mla_decode_fwd(q[..., :512].contiguous(), kv, idx, 1.0)
    with pytest.raises(ValueError, match="does not go with"):
        smla.flash_ops.sparse_mla_prefill_fwd(q, kv_m1, idx, 1.0)
    with pytest.raises(ValueError, match="layout of the main cache"):
        smla.flash_ops.sparse_mla_decode_fwd(q, kv, idx, 1.0, extra_k_cache=kv_m1, extra_indices=idx, extra_topk=64)
    with pytest.raises(ValueError, match="needs extra_k_cache"):
        smla.flash_ops.sparse_mla_decode_fwd(q, kv, idx, 1.0, extra_topk=64)


def test_model1_default_impl():
    """IMPL_AUTO resolves per layout: the tensor-core kernel for 656-byte rows, the exact fp32 kernel for MODEL1
    unless the module switch says otherwise; an explicit choice is never changed."""
    from sparse_mla_sm120_b200 import _runtime
    L = _lib
    assert _runtime.resolve_impl(L.IMPL_AUTO, L.LAYOUT_V32) == L.IMPL_AUTO
    assert _runtime.resolve_impl(L.IMPL_AUTO, L.LAYOUT_MODEL1) == _runtime.MODEL1_DEFAULT_IMPL == L.IMPL_SCALAR
    assert _runtime.resolve_impl(L.IMPL_TC, L.LAYOUT_MODEL1) == L.IMPL_TC
    assert _runtime.resolve_impl(L.IMPL_SCALAR, L.LAYOUT_V32) == L.IMPL_SCALAR


def test_split_policy():
    from sparse_mla_sm120_b200._runtime import FIXED_OVERHEAD, pick_num_sm_parts, pick_split
    # lengths unknown or different: the general rule
    assert pick_num_sm_parts(64, 148) == 64      # 128 CTAs on 148 SMs: unsplit
    assert pick_num_sm_parts(128, 148) == 128    # two nearly full waves: unsplit
    assert pick_num_sm_parts(40, 148) == 40      # more than half of the machine: unsplit
    assert pick_num_sm_parts(1, 148) == 74       # small batch, top-k unknown: cut into sms/2 partitions
    assert pick_num_sm_parts(36, 148) == 74
    # with the top-k known, no partition gets fewer than four 64-token blocks
    assert pick_num_sm_parts(1, 148, 32) == 8
    assert pick_num_sm_parts(4, 148, 32) == 32
    assert pick_num_sm_parts(16, 148, 32) == 74
    assert pick_num_sm_parts(4, 148, 1) == 4     # nothing worth splitting: one partition per request, attention kernel alone
    assert pick_split(16, 148, 32, uniform=False) == (74, FIXED_OVERHEAD)
    # requests of equal length: k equal partitions each (fixed overhead 0 keeps them from straddling two requests)
    assert pick_split(1, 148, 32, uniform=True) == (8, 0)
    assert pick_split(8, 148, 32, uniform=True) == (64, 0)
    assert pick_split(12, 148, 32, uniform=True) == (48, 0)    # four partitions each: eight would not fit the machine
    assert pick_split(16, 148, 32, uniform=True) == (64, 0)
    assert pick_split(32, 148, 32, uniform=True) == (64, 0)
    assert pick_split(37, 148, 32, uniform=True) == (74, 0)    # two partitions each still fit the machine
    assert pick_split(40, 148, 32, uniform=True)[0] == 40      # unsplit
    assert pick_split(64, 148, 32, uniform=True)[0] == 64
    assert pick_split(128, 148, 32, uniform=True)[0] == 128
    assert pick_split(4, 148, 8, uniform=True)[0] == 4         # short requests: not worth the scheduler and combine launches
    assert pick_split(4, 148, 31, uniform=True) == (31, FIXED_OVERHEAD)   # no divisor: the general rule


def test_flashmla_surface_argument_checks():
    """The FlashMLA-shaped wrappers refuse what the reference refuses, before any device work."""
    import pytest
    import torch
    from sparse_mla_sm120_b200 import interface
    meta, none = interface.get_mla_metadata()
    assert none is None and isinstance(meta, interface.FlashMLASchedMeta) and not meta.have_initialized
    q = torch.zeros(1, 1, 128, 576, dtype=torch.bfloat16)
    kv = torch.zeros(2, 64, 1, 656, dtype=torch.uint8)
    idx = torch.zeros(1, 1, 64, dtype=torch.int32)
    with pytest.raises(TypeError):
        interface.flash_mla_with_kvcache(q, kv, None, None, 512, object(), None, None, False, True, indices=idx)
    with pytest.raises(ValueError):
        interface.flash_mla_with_kvcache(q, kv, None, None, 512, meta, None, None, False, True, indices=None)
    with pytest.raises(ValueError):
        interface.flash_mla_with_kvcache(q, kv, None, None, 512, meta, None, None, False, False, indices=idx)
    with pytest.raises(ValueError):    # no CPU path
        interface.flash_mla_with_kvcache(q, kv, None, None, 512, meta, None, None, False, True, indices=idx)
    assert not meta.have_initialized
