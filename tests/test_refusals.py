"""Sizes and arguments the kernels do not take are refused by their entry points with a status, before
anything is launched: checked here on the CPU (the libraries load without a GPU; a refused call touches
no CUDA function). -1: element type, -2: size, -3: alignment, -4: missing or contradictory argument."""
import ctypes

import pytest

from cellm_b200.ops import _lib

BUF = ctypes.create_string_buffer(4096)
A = (ctypes.addressof(BUF) + 255) & ~255        # a 256-byte aligned address that no refused call reads
DTYPE, SIZE, ALIGN, ARG = -1, -2, -3, -4


def call(library, name, *args):
    return _lib.fn(library, name)(*args)


def gemm(M=8, N=256, K=64, lda=None, ldw=None, out=1, bn=-16, split=1, epi=0, a=A, w=A):
    return call("gemm_tcgen05", "cellm_gemm_tcgen05", A, a, w, M, N, K, lda or K, ldw or K, N, out, bn, split, epi, 0,
                None, None, A, None)


def test_tensor_core_product():
    assert gemm(K=100) == SIZE and gemm(K=0) == SIZE                      # K must be a positive multiple of 8
    assert gemm(a=A + 2) == ALIGN and gemm(w=A + 8) == ALIGN and gemm(lda=68) == ALIGN
    assert gemm(out=2) == DTYPE
    assert gemm(bn=-48) == SIZE and gemm(bn=96) == SIZE and gemm(bn=0) == SIZE
    assert gemm(epi=1, N=192) == SIZE and gemm(epi=1, N=256, bn=64) == SIZE      # SwiGLU: blocks of 128, tiles of >= 128
    assert gemm(epi=2) == ARG and gemm(epi=3) == ARG and gemm(epi=7) == ARG       # those have entry points of their own
    assert gemm(M=0) == 0 and gemm(N=0) == 0                                     # nothing to do


def test_product_with_the_convolution_in_its_epilogue():
    def conv(M=8, Nt=384, K=64, H=100, bn=-16, taps=A, ntaps=3, state=A, slots=A, n_slots=4):
        return call("gemm_tcgen05", "cellm_gemm_conv_tcgen05", A, A, A, M, Nt, K, K, K, H, bn, 1, taps, None, ntaps, state,
                    200, slots, n_slots, 1, A, None)
    assert conv(Nt=400) == SIZE            # tiles of 128 rows
    assert conv(Nt=256) == SIZE            # two tiles hold 84 channels, not 100
    assert conv(bn=128) == SIZE and conv(H=0) == SIZE
    assert conv(ntaps=5) == SIZE and conv(ntaps=0) == SIZE
    assert conv(taps=None) == ARG and conv(slots=None) == ARG and conv(state=None) == ARG and conv(n_slots=0) == ARG
    assert conv(M=0) == 0


def test_product_with_the_rotation_in_its_epilogue():
    def rope(M=4, K=64, bn=-16, q_w=A, k_w=A, pos=A, bt=A, stride=8, kp=A, vp=A, pages=4, ps=16, nh=4, nkv=2, inv=A):
        return call("gemm_tcgen05", "cellm_gemm_rope_tcgen05", A, A, A, M, K, K, K, bn, 1, q_w, k_w, 1e-5, pos, bt, stride,
                    kp, vp, pages, ps, nh, nkv, inv, 1, A, None)
    assert rope(bn=64) == SIZE and rope(nh=0) == SIZE and rope(nkv=0) == SIZE and rope(ps=0) == SIZE and rope(stride=0) == SIZE
    for missing in ("q_w", "k_w", "pos", "bt", "kp", "vp", "inv"):
        assert rope(**{missing: None}) == ARG
    assert rope(M=0) == 0


def test_attention_kernels():
    def decode(nh=4, nkv=2, hd=64, nsplit=1, part=None, counters=None):
        return call("attention_decode", "cellm_attention_decode", A, part, part, counters, A, A, A, A, A, A, 4, 2, 2, 8, 16,
                    nh, nkv, hd, 0.125, 0, nsplit, A, None)
    assert decode(nh=5) == SIZE and decode(nkv=0) == SIZE and decode(nh=34, nkv=2) == SIZE      # at most 16 heads a group
    assert decode(hd=48) == SIZE and decode(hd=256) == SIZE
    assert decode(nsplit=0) == ARG and decode(nsplit=9) == ARG and decode(nsplit=9, part=A) == ARG      # more pieces than a cluster: workspace and counters

    def flash(nh=4, nkv=2, hd=64, nsplit=1, part=None):
        return call("attention_flash", "cellm_attention_flash", A, part, part, A, A, A, A, A, A, 4, 2, 8, 1, 8, 16, nh, nkv, hd,
                    0.125, 0, 1, nsplit, A, None)
    assert flash(nh=5) == SIZE and flash(hd=80) == SIZE and flash(nsplit=2) == ARG and flash(nsplit=0) == ARG
    supports = _lib.fn("attention_flash", "cellm_attention_flash_supports")
    assert [supports(hd) for hd in (16, 32, 48, 64, 128, 256)] == [0, 1, 0, 1, 1, 0]

    tc_supports = _lib.fn("attention_tc", "cellm_attention_tc_supports")
    assert tc_supports(64, 32, 8, 16) == 1 and tc_supports(128, 32, 8, 16) == 0 and tc_supports(64, 6, 2, 16) == 0
    assert tc_supports(64, 32, 8, 4) == 0 and tc_supports(64, 32, 8, 24) == 0

    def tc(hd=64, nh=32, nkv=8, ps=16, scale=0.125, q=A):
        return call("attention_tc", "cellm_attention_tc", A, q, A, A, A, A, A, 4, 1, 8, 1, 8, ps, nh, nkv, hd, scale, 0, A, None)
    assert tc(hd=128) == SIZE and tc(ps=4) == SIZE and tc(scale=0.0) == SIZE and tc(q=A + 4) == ALIGN

    def plain(nh=4, nkv=2, hd=64):
        return call("kernels_common", "cellm_attention_plain", A, A, A, A, A, A, A, 4, 8, 16, 2, nh, nkv, hd, 0.125, 0, 1, A, None)
    assert plain(hd=520) == SIZE and plain(hd=0) == SIZE and plain(nh=5) == SIZE


def test_small_kernels():
    def conv(taps):
        return call("kernels_common", "cellm_short_conv", A, A, A, None, 1, A, 64, A, A, A, 2, 1, 16, taps, 2, 1, 1, A, None)
    assert conv(0) == SIZE and conv(17) == SIZE

    def rope(rot=64, hd=64, q_w=A, k_w=A):
        return call("kernels_common", "cellm_qk_norm_rope", A, A, 256, q_w, k_w, 1, 1e-5, A, A, None, 0, None, None, 0, 16, 2,
                    2, 0, hd, rot, 0, A, 1, A, None)
    assert rope(rot=66) == SIZE and rope(rot=31) == SIZE and rope(rot=-2) == SIZE
    assert rope(q_w=None) == ARG and rope(k_w=None) == ARG

    def sample(W=0, k=40):
        return call("kernels_common", "cellm_sample", A, A, 2, 1000, A, A, A, None, None, W, k, None, None)
    assert sample(k=1025) == SIZE and sample(W=257) == SIZE and sample(W=-1) == SIZE
    assert call("gemm_plain", "cellm_gemm_plain", A, A, A, 2, 4, 0, 8, 8, 4, 1, 1, None) == SIZE
