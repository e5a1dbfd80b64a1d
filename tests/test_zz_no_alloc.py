"""The allocation-free arg-max entry point, called through its exported C symbol.

It exists for hosts that cannot get device memory when they call (no PyTorch allocator in the
process, all HBM already promised to the KV cache, or a stream capture in progress), so its
scratch space is a fixed array inside the library.  Here it must agree with the ordinary entry
point `sl_argmax`, on two calls in a row (the second call finds the first one's leftovers in the
array) and reject a batch larger than the built-in scratch without launching anything.
The file name sorts last so that a run that stops at the first failure has already covered
every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from slopllm_b200.ops import native as N
    lib = N.kernels()
    lib.sl_argmax_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_void_p,
                                      C.c_void_p]
    lib.sl_argmax_noalloc.restype = C.c_int
    return lib


def _existing(logits, offset=0):
    from slopllm_b200.config import GlmMoeDsaConfig
    from slopllm_b200.ops.cuda_ops import CudaOps
    return CudaOps(GlmMoeDsaConfig.tiny()).argmax(logits, id_offset=offset, want_val=True)


def test_noalloc_argmax_matches_existing_entry_point_twice():
    lib = _lib()
    dev = "cuda"
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=dev).manual_seed(7)
    for call, (rows, vocab, dtype) in enumerate([(8, 154880, torch.float32), (3, 4099, torch.bfloat16)]):
        logits = torch.randn(rows, vocab + 5, device=dev, generator=g).to(dtype)[:, :vocab]      # ld > vocab
        logits[0, 10] = logits[0, 20] = 99.0                                                        # tie -> lower index
        out = torch.full((rows,), -1, dtype=torch.int64, device=dev)
        val = torch.zeros(rows, dtype=torch.float32, device=dev)
        rc = lib.sl_argmax_noalloc(out.data_ptr(), logits.data_ptr(), rows, vocab, logits.stride(0),
                                   int(dtype == torch.float32), 1000 * call, val.data_ptr(), stream)
        assert rc == 0
        ids, vals = _existing(logits, 1000 * call)
        torch.cuda.synchronize()
        assert torch.equal(out, ids)
        assert torch.allclose(val, vals, rtol=1e-2, atol=1e-2)
        assert int(out[0]) == 10 + 1000 * call
        assert torch.equal(out - 1000 * call, logits.float().argmax(-1))


def test_noalloc_argmax_rejects_oversize_and_bad_arguments():
    lib = _lib()
    x = torch.zeros(4, 16, device="cuda")
    out = torch.zeros(4, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.sl_argmax_noalloc(out.data_ptr(), x.data_ptr(), 257, 16, 16, 1, 0, None, stream) == -22
    assert lib.sl_argmax_noalloc(out.data_ptr(), x.data_ptr(), 4, 16, 8, 1, 0, None, stream) == -23
    assert lib.sl_argmax_noalloc(None, x.data_ptr(), 4, 16, 16, 1, 0, None, stream) == -23
    torch.cuda.synchronize()


def _call(lib, logits, offset=0, want_val=True):
    rows, vocab = logits.shape
    out = torch.full((rows,), -7, dtype=torch.int64, device=logits.device)
    val = torch.zeros(rows, dtype=torch.float32, device=logits.device) if want_val else None
    rc = lib.sl_argmax_noalloc(out.data_ptr(), logits.data_ptr(), rows, vocab, logits.stride(0),
                               int(logits.dtype == torch.float32), offset, val.data_ptr() if want_val else None,
                               torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, out, val


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_argmax_ties_across_chunks_and_at_the_row_end(dtype):
    """Equal maxima in different chunks of the 64-way split (index 5 and the last index) resolve to the lower index,
    and a maximum that only the very last element holds is found."""
    lib = _lib()
    g = torch.Generator(device="cuda").manual_seed(11)
    vocab = 154880
    x = torch.randn(3, vocab, device="cuda", generator=g).to(dtype)
    x[0, 5] = x[0, vocab - 1] = 50.0
    x[1, vocab - 1] = 60.0
    x[2, vocab // 2] = x[2, vocab // 2 + 1] = 70.0          # neighbours inside one chunk
    rc, out, val = _call(lib, x)
    assert rc == 0
    assert out.tolist() == [5, vocab - 1, vocab // 2]
    assert val.tolist() == [50.0, 60.0, 70.0]


def test_noalloc_argmax_full_scratch_with_small_vocab():
    """The largest batch the built-in scratch takes, with fewer columns than the 64 chunks of a row (most chunks are
    empty and must still leave a defined partial), against torch."""
    lib = _lib()
    g = torch.Generator(device="cuda").manual_seed(12)
    for vocab in (1, 7, 63, 64, 65, 130):
        x = torch.randn(256, vocab, device="cuda", generator=g)
        rc, out, val = _call(lib, x, offset=3)
        assert rc == 0
        assert torch.equal(out - 3, x.argmax(-1))
        assert torch.equal(val, x.max(-1).values)


def test_noalloc_argmax_rows_without_a_finite_maximum():
    """A row of NaN only, a row of -inf only and a row mixing both give index 0 (+ offset), like `sl_argmax`; a NaN
    next to finite values is skipped."""
    lib = _lib()
    vocab = 4099
    x = torch.zeros(4, vocab, device="cuda")
    x[0] = float("nan")
    x[1] = float("-inf")
    x[2] = float("-inf")
    x[2, ::2] = float("nan")
    x[3] = torch.arange(vocab, device="cuda", dtype=torch.float32) * -1.0
    x[3, 17] = float("nan")
    x[3, 99] = 5.0
    rc, out, val = _call(lib, x, offset=100)
    assert rc == 0
    assert out.tolist() == [100, 100, 100, 199]
    ids, _ = _existing(x, 100)
    assert torch.equal(out, ids)
    assert float(val[3]) == 5.0 and float(val[1]) == float("-inf")
