"""mk36_full_attention_decode_static: the attention decode entry point that keeps its scratch in a
fixed device array inside the library and allocates nothing.

Called through the C ABI (ctypes, raw device pointers) and compared with the workspace-taking
entry point mk36_full_attention_decode on the same inputs.  The file sorts last on purpose: the
static array is shared by every call in the process, so this also shows the entry point working
after whatever the other tests left behind, as well as on its own.
"""

import pytest
import torch

import parity

pytestmark = pytest.mark.gpu


def _tensors(dev, batch, hq, hkv, d, t, seed, dtype=torch.bfloat16):
    from mega_kernel_qwen36 import synthetic as syn

    return {k: v.to(dev).contiguous() for k, v in syn.attention_tensors(batch, hq, hkv, d, t, seed=seed, dtype=dtype).items()}


def _args(cabi, t, out, batch, hq, hkv, d, seq, dtype_code):
    return cabi.AttentionArgs(q=t["q"].data_ptr(), k_cache=t["k_cache"].data_ptr(), v_cache=t["v_cache"].data_ptr(),
                              out=out.data_ptr(), dtype=dtype_code, batch=batch, query_heads=hq, kv_heads=hkv,
                              head_dim=d, seq_len=seq, scale=float(d) ** -0.5)


def _with_workspace(cabi, lib, t, shape, dtype_code, stream):
    out = torch.empty_like(t["q"])
    args = _args(cabi, t, out, *shape, dtype_code)
    nbytes = lib.mk36_attention_workspace_bytes(args)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=out.device)
    cabi.check(lib.mk36_workspace_init(ws.data_ptr(), nbytes, stream))
    cabi.check(lib.mk36_full_attention_decode(args, ws.data_ptr(), nbytes, stream))
    torch.cuda.synchronize()
    return out


# (batch, query heads, kv heads, head_dim, cached tokens): the 35B-A3B head layout at two cache
# lengths, then a shape only the general (non tensor-core) kernel takes (fp32).
CASES = [
    ((1, 16, 2, 256, 4096), torch.bfloat16, 11),
    ((2, 16, 2, 256, 777), torch.bfloat16, 12),
    ((3, 8, 2, 64, 513), torch.float32, 13),
]


def test_static_scratch_entry_matches_workspace_entry_on_consecutive_calls(cuda_device):
    from mega_kernel_qwen36 import cabi

    lib = cabi.load()
    stream = torch.cuda.current_stream().cuda_stream
    codes = {torch.bfloat16: cabi.MK36_BF16, torch.float16: cabi.MK36_F16, torch.float32: cabi.MK36_F32}
    # every call below goes to the same built-in array, back to back on one stream, with different
    # shapes and therefore different scratch layouts: nothing a call leaves behind may leak into the next
    for shape, dtype, seed in CASES:
        t = _tensors(cuda_device, *shape, seed=seed, dtype=dtype)
        expect = _with_workspace(cabi, lib, t, shape, codes[dtype], stream)
        outs = []
        for _ in range(2):
            out = torch.full_like(t["q"], float("nan"))
            cabi.check(lib.mk36_full_attention_decode_static(_args(cabi, t, out, *shape, codes[dtype]), stream))
            outs.append(out)
        torch.cuda.synchronize()
        for i, out in enumerate(outs):
            parity.assert_output_parity(out.cpu(), expect.cpu(), f"static call {i} {shape}")
        # same kernels, same split plan: in fact the results are identical
        assert torch.equal(outs[0], outs[1])
        assert torch.equal(outs[0], expect)


def test_static_scratch_entry_two_problems_in_a_row_without_sync(cuda_device):
    """Two different problems queued back to back on one stream share the array in stream order."""
    from mega_kernel_qwen36 import cabi

    lib = cabi.load()
    stream = torch.cuda.current_stream().cuda_stream
    shape_a, shape_b = (1, 16, 2, 256, 2048), (4, 16, 4, 128, 300)
    ta, tb = _tensors(cuda_device, *shape_a, seed=21), _tensors(cuda_device, *shape_b, seed=22)
    ea = _with_workspace(cabi, lib, ta, shape_a, cabi.MK36_BF16, stream)
    eb = _with_workspace(cabi, lib, tb, shape_b, cabi.MK36_BF16, stream)
    oa, ob = torch.empty_like(ta["q"]), torch.empty_like(tb["q"])
    cabi.check(lib.mk36_full_attention_decode_static(_args(cabi, ta, oa, *shape_a, cabi.MK36_BF16), stream))
    cabi.check(lib.mk36_full_attention_decode_static(_args(cabi, tb, ob, *shape_b, cabi.MK36_BF16), stream))
    torch.cuda.synchronize()
    parity.assert_output_parity(oa.cpu(), ea.cpu(), "first queued problem")
    parity.assert_output_parity(ob.cpu(), eb.cpu(), "second queued problem")


def test_static_scratch_entry_argument_errors(cuda_device):
    from mega_kernel_qwen36 import cabi

    lib = cabi.load()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.mk36_full_attention_decode_static(None, stream) == cabi.MK36_ERR_INVALID_ARG
    shape = (1, 16, 2, 256, 64)
    t = _tensors(cuda_device, *shape, seed=3)
    out = torch.empty_like(t["q"])
    args = _args(cabi, t, out, *shape, cabi.MK36_BF16)
    args.kv_heads = 3  # 16 query heads do not divide over 3 kv heads: refused before any launch
    assert lib.mk36_full_attention_decode_static(args, stream) != cabi.MK36_OK
    assert lib.mk36_last_error()
    # the device stays usable and the next good call works
    args.kv_heads = 2
    cabi.check(lib.mk36_full_attention_decode_static(args, stream))
    torch.cuda.synchronize()
    expect = _with_workspace(cabi, lib, t, shape, cabi.MK36_BF16, stream)
    assert torch.equal(out, expect)


def test_static_scratch_entry_refuses_what_does_not_fit_and_writes_nothing(cuda_device):
    """A plan that needs more scratch than the array is refused before anything is launched: the
    call returns MK36_ERR_WORKSPACE, names the limit, and leaves `out` as it was.  The array is
    made to look small ("static_scratch_limit") so that a modest problem is enough, once for a
    single-launch call and once for a batch that would need several launches."""
    from mega_kernel_qwen36 import cabi

    lib = cabi.load()
    stream = torch.cuda.current_stream().cuda_stream
    cabi.check(lib.mk36_set_option(b"static_scratch_limit", 48 * 1024))
    try:
        for shape in ((1, 16, 2, 256, 4096), (96, 16, 2, 256, 512)):
            t = _tensors(cuda_device, *shape, seed=31)
            out = torch.full_like(t["q"], 7.0)
            rc = lib.mk36_full_attention_decode_static(_args(cabi, t, out, *shape, cabi.MK36_BF16), stream)
            torch.cuda.synchronize()
            assert rc == cabi.MK36_ERR_WORKSPACE, (shape, rc)
            assert b"built-in" in lib.mk36_last_error()
            assert bool((out == 7.0).all()), f"{shape}: a refused call wrote to out"
    finally:
        cabi.check(lib.mk36_set_option(b"static_scratch_limit", 0))
    # with the full array the first problem fits again and matches the workspace variant
    shape = (1, 16, 2, 256, 4096)
    t = _tensors(cuda_device, *shape, seed=31)
    out = torch.empty_like(t["q"])
    cabi.check(lib.mk36_full_attention_decode_static(_args(cabi, t, out, *shape, cabi.MK36_BF16), stream))
    torch.cuda.synchronize()
    assert torch.equal(out, _with_workspace(cabi, lib, t, shape, cabi.MK36_BF16, stream))


def test_static_scratch_status_reads_the_word_in_the_array(cuda_device):
    """The status word of the static calls lives in the array; the accessor reports it (clean here)."""
    import ctypes

    from mega_kernel_qwen36 import cabi

    lib = cabi.load()
    stream = torch.cuda.current_stream().cuda_stream
    shape = (2, 16, 2, 128, 700)
    t = _tensors(cuda_device, *shape, seed=5)
    out = torch.empty_like(t["q"])
    cabi.check(lib.mk36_full_attention_decode_static(_args(cabi, t, out, *shape, cabi.MK36_BF16), stream))
    status = ctypes.c_int(-1)
    cabi.check(lib.mk36_static_scratch_status(stream, ctypes.byref(status)))
    assert status.value == 0
    assert lib.mk36_static_scratch_status(stream, None) == cabi.MK36_ERR_INVALID_ARG
