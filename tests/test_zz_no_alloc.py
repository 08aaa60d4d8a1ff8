"""The attention entry point that allocates nothing, called through its
exported C symbol, against the regular entry point.

Some users of the library cannot ask for device memory when they need a result
(a callback that must not enter the driver's allocator, a host application
that handed the engine a fixed arena). For them `cellm_attention_flash_noalloc`
keeps the pieces of a key split in an array inside the library itself. This
test calls it twice in a row with different inputs, so that a second call that
trusted what the first left in the shared array would show, and checks that an
oversized call is refused before anything is launched.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(q_lens, ctx_lens, nh, nkv, hd, ps, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    dev = "cuda:0"
    B = len(q_lens)
    totals = [c + n for c, n in zip(ctx_lens, q_lens)]
    nblk = [(t + ps - 1) // ps for t in totals]
    pages = sum(nblk) + 2
    perm = torch.randperm(pages, generator=g).tolist()
    bt = torch.full((B, max(nblk)), -1, dtype=torch.int32)
    o = 0
    for b in range(B):
        bt[b, :nblk[b]] = torch.tensor(perm[o:o + nblk[b]], dtype=torch.int32)
        o += nblk[b]
    mk = lambda *s: torch.randn(*s, generator=g).to(dev).bfloat16()
    cu = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
    return dict(q=mk(sum(q_lens), nh * hd), k=mk(pages, nkv, ps, hd), v=mk(pages, nkv, ps, hd), cu=cu,
                ctx=torch.tensor(ctx_lens, dtype=torch.int32, device=dev), bt=bt.to(dev), q_lens=q_lens, nh=nh)


def _call_noalloc(lib, x, nsplit, wide, err):
    f = lib.cellm_attention_flash_noalloc
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    f.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, I, I, P, P]
    f.restype = I
    pages, nkv, ps, hd = x["k"].shape
    T, nh = x["q"].shape[0], x["nh"]
    G = nh // nkv
    bm = 64 if wide else 16
    n_tiles = sum((n * G + bm - 1) // bm for n in x["q_lens"])
    out = torch.empty_like(x["q"])
    rc = f(out.data_ptr(), x["q"].data_ptr(), x["k"].data_ptr(), x["v"].data_ptr(), x["cu"].data_ptr(),
           x["ctx"].data_ptr(), x["bt"].data_ptr(), x["bt"].stride(0), len(x["q_lens"]), T, n_tiles, pages, ps, nh,
           nkv, hd, 1.0 / math.sqrt(hd), 0, 1 if wide else 0, nsplit, err.data_ptr(),
           torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_no_alloc_entry_point_matches_regular_entry_point():
    from cellm_b200.csrc import build
    from cellm_b200.ops.attention import attention_flash
    lib = build.load("attention_flash")
    lib.cellm_attention_flash_noalloc_error.restype = ctypes.c_char_p
    lib.cellm_attention_flash_noalloc_capacity.restype = ctypes.c_longlong
    assert lib.cellm_attention_flash_noalloc_capacity() == 2 * 1024 * 1024
    err = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    cases = [(_inputs([1, 1, 1], [300, 40, 513], 8, 2, 64, 16, seed=1), 4, False),
             (_inputs([70, 1], [130, 900], 6, 2, 32, 8, seed=2), 3, True),
             (_inputs([33, 5], [0, 77], 4, 4, 128, 16, seed=4), 1, True),           # one piece: the array is not used at all
             # the largest call that fits: 4 pieces x 992 tokens x 8 heads x 66 floats = 2,095,104 of 2,097,152
             (_inputs([992], [0], 8, 2, 64, 16, seed=5), 4, True)]
    for x, nsplit, wide in cases:        # two calls in a row on the one shared array
        ref = attention_flash(x["q"], x["k"], x["v"], x["cu"], x["ctx"], x["bt"], x["q_lens"], x["nh"],
                              1.0 / math.sqrt(x["k"].shape[3]), 0, err, nsplit, wide)
        rc, out = _call_noalloc(lib, x, nsplit, wide, err)
        assert rc == 0, lib.cellm_attention_flash_noalloc_error(rc).decode()
        torch.cuda.synchronize()
        assert err.item() == 0
        # same kernels, same order of sums: the two entry points agree to the last bit
        assert torch.equal(out, ref)
        # and both agree with the plain kernel within bfloat16 rounding of the output
        from cellm_b200.ops.basic import attention_plain
        pos = torch.cat([torch.arange(c, c + n) for c, n in zip(x["ctx"].tolist(), x["q_lens"])]).int().cuda()
        seq = torch.cat([torch.full((n,), b) for b, n in enumerate(x["q_lens"])]).int().cuda()
        plain = attention_plain(x["q"], x["k"], x["v"], pos, seq, x["bt"], x["nh"], 1.0 / math.sqrt(x["k"].shape[3]), 0, err)
        assert (out.float() - plain.float()).abs().max().item() <= 2e-2 * (1 + plain.float().abs().max().item())


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from cellm_b200.csrc import build
    lib = build.load("attention_flash")
    lib.cellm_attention_flash_noalloc_error.restype = ctypes.c_char_p
    err = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    x = _inputs([600], [0], 32, 8, 128, 16, seed=3)      # 8 * 600 * 32 * 130 floats > 2 Mi
    rc, _ = _call_noalloc(lib, x, 8, True, err)
    assert rc == -5
    assert b"scratch" in lib.cellm_attention_flash_noalloc_error(rc)
    rc, _ = _call_noalloc(lib, x, 0, True, err)
    assert rc == -4
    # one token more than the largest call that fits (see the test above) is refused
    rc, _ = _call_noalloc(lib, _inputs([993], [0], 8, 2, 64, 16, seed=5), 4, True, err)
    assert rc == -5
    # a head size the kernel does not take reads as that, whatever the pieces would need
    bad = _inputs([600], [0], 32, 8, 48, 16, seed=6)
    rc, _ = _call_noalloc(lib, bad, 8, True, err)
    assert rc == -2
    torch.cuda.synchronize()
    assert err.item() == 0
