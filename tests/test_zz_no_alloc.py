"""The decode-attention entry point that allocates nothing (csrc/attention_noalloc.h).

Some users of this library cannot allocate device memory at the moment they need attention: their
code is a plug-in in an application that owns the GPU's memory, or it runs in a loop that must stay
clear of the allocator.  For them the library carries its own fixed scratch array, and
``pe_attention_decode_noalloc`` takes inputs and outputs only.  This test calls that function
through its exported C symbol, twice in a row with different batches (the array keeps the first
call's contents, which must not leak into the second), and compares each result with the ordinary
entry point, which is given scratch memory by the caller.  It also checks that a call too large for
the built-in array is refused.  The file sorts last so that a run that stops at the first failure
has run every other test before it.
"""
import ctypes
import math
import os
import re

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _header_constant(pe, name):
    header = os.path.join(os.path.dirname(pe.kernels.build.CSRC + "/"), "attention_noalloc.h")
    text = open(header).read()
    m = re.search(rf"#define\s+{name}\s+\((.+?)\)", text)
    return int(eval(m.group(1).replace("<<", "<<")))  # "1 << 21" or "-6"


def _case(seed, lens, nh, nkv, d, dtype):
    from test_kernels_gpu import PagedSetup
    ps = PagedSetup(lens, nkv, d, dtype, seed=seed, key_scale=2.0)
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(len(lens), nh * d, generator=g).to(dtype).to(DEV)
    qstart = torch.arange(len(lens) + 1, dtype=torch.int32, device=DEV)
    past = torch.tensor([L - 1 for L in lens], dtype=torch.int32, device=DEV)
    return ps, q, qstart, past


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_entry_point_matches_the_ordinary_one(pe, dtype):
    lib = pe.kernels.library()
    ops = pe.kernels.ops
    fn = lib.pe_attention_decode_noalloc          # the exported C symbol
    nh, nkv, d, split, max_splits = 8, 2, 64, 256, 3
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    for seed, lens in [(1, [700, 5, 256, 257]), (2, [33, 300])]:      # two calls in a row; the second is smaller
        ps, q, qstart, past = _case(seed, lens, nh, nkv, d, dtype)
        B = len(lens)
        want = torch.zeros(B, nh * d, device=DEV, dtype=dtype)
        scratch = torch.zeros(ops.attention_generic_scratch_floats(B, nh, d, max_splits), device=DEV)
        ops.attention_generic(True, q, want, B, 1, nh, nkv, d, 1 / math.sqrt(d), 0, qstart, past, ps.seq_slot, ps.table,
                              ps.num_pages, ps.k_pages, ps.v_pages, scratch, split, max_splits, status)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        rc = fn(ops.dtype_tag(dtype), q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), B, nh, nkv, d,
                ctypes.c_float(1 / math.sqrt(d)), 0, qstart.data_ptr(), past.data_ptr(), ps.seq_slot.data_ptr(),
                ps.table.data_ptr(), ps.table.shape[1], ps.num_pages, ps.k_pages.data_ptr(), ps.v_pages.data_ptr(),
                split, max_splits, status.data_ptr(), stream)
        torch.cuda.synchronize()
        assert rc == 0
        assert status.tolist()[0] == 0
        tol = 5e-6 if dtype == torch.float32 else 8e-3           # the attention tests' tolerance
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err < tol, (lens, err)


def test_no_alloc_entry_point_refuses_what_does_not_fit(pe):
    lib = pe.kernels.library()
    limit = _header_constant(pe, "PE_NOALLOC_SCRATCH_FLOATS")
    too_large = _header_constant(pe, "PE_ERR_SCRATCH_TOO_LARGE")
    nh, d, max_splits = 32, 128, 16
    n_seqs = limit // (nh * max_splits * (d + 1)) + 1
    z = torch.zeros(8, device=DEV)
    rc = lib.pe_attention_decode_noalloc(0, z.data_ptr(), nh * d, z.data_ptr(), nh * d, n_seqs, nh, 8, d,
                                         ctypes.c_float(1.0), 0, z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, 1,
                                         z.data_ptr(), z.data_ptr(), 256, max_splits, z.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == too_large
    with pytest.raises(pe.kernels.KernelError, match="scratch"):
        pe.kernels.lib.check(rc, "pe_attention_decode_noalloc")


def test_a_sequence_longer_than_its_ranges_sets_the_status_word(pe):
    """``max_splits`` ranges of ``split_keys`` keys must cover every sequence.  The lengths are on the device, so
    the kernel checks: a longer sequence sets the status word and is merged over the ranges that exist (no read
    beyond the scratch).  The same check guards the ordinary entry point and the tensor-core one."""
    lib = pe.kernels.library()
    ops = pe.kernels.ops
    nh, nkv, d, split, max_splits = 8, 2, 64, 256, 2
    stream = torch.cuda.current_stream().cuda_stream
    lens = [700, 40]                                     # 700 > 2 * 256
    for dtype in (torch.float32, torch.bfloat16):
        ps, q, qstart, past = _case(5, lens, nh, nkv, d, dtype)
        B = len(lens)
        # what the first 512 keys alone give: the same call on a sequence cut to 512 keys
        past_cut = torch.tensor([511, 39], dtype=torch.int32, device=DEV)
        want = torch.zeros(B, nh * d, device=DEV, dtype=dtype)
        status = torch.zeros(4, dtype=torch.int32, device=DEV)
        scratch = torch.zeros(ops.attention_generic_scratch_floats(B, nh, d, max_splits), device=DEV)
        args = (B, 1, nh, nkv, d, 1 / math.sqrt(d), 0, qstart)
        tail = (ps.seq_slot, ps.table, ps.num_pages, ps.k_pages, ps.v_pages, scratch, split, max_splits, status)
        ops.attention_generic(True, q, want, *args, past_cut, *tail)
        assert status.tolist()[0] == 0
        kernels = [lambda out: ops.attention_generic(True, q, out, *args, past, *tail)]
        if dtype == torch.bfloat16:
            kernels.append(lambda out: ops.attention_mma(True, q, out, *args, past, *tail))
        kernels.append(lambda out: pe.kernels.lib.check(lib.pe_attention_decode_noalloc(
            ops.dtype_tag(dtype), q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), B, nh, nkv, d,
            ctypes.c_float(1 / math.sqrt(d)), 0, qstart.data_ptr(), past.data_ptr(), ps.seq_slot.data_ptr(),
            ps.table.data_ptr(), ps.table.shape[1], ps.num_pages, ps.k_pages.data_ptr(), ps.v_pages.data_ptr(),
            split, max_splits, status.data_ptr(), stream), "noalloc"))
        for run in kernels:
            status.zero_()
            got = torch.full_like(want, float("nan"))
            run(got)
            torch.cuda.synchronize()
            assert status.tolist() == [3, 0, 699, 512]
            assert torch.isfinite(got.float()).all()
            # the long sequence got the attention over the keys its ranges cover; the short one is untouched
            for row in (0, 1):
                err = float((got[row].float() - want[row].float()).abs().max() / want[row].float().abs().max())
                assert err < (5e-6 if dtype == torch.float32 else 8e-3), (row, err)
