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
