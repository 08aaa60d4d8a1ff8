"""Each kernel alone against a plain float32/float64 torch restatement of the
same operation, at sizes other than the engine's (widths that are no power of
two, odd counts, several head sizes and page sizes)."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = [torch.float32, torch.bfloat16]


def tol(dtype, ref):
    k = 2e-6 if dtype == torch.float32 else 1.2e-2
    return k * (1.0 + float(ref.abs().max()))


def close(got, ref, dtype, what=""):
    assert got.shape == ref.shape, f"{what}: {tuple(got.shape)} against {tuple(ref.shape)}"
    if ref.numel() == 0:            # a convolution of one tap carries no state
        return
    err = float((got.double().cpu() - ref.double().cpu()).abs().max())
    assert err <= tol(dtype, ref.double()), f"{what}: {err} > {tol(dtype, ref.double())}"


def err_word():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", DT)
def test_embed(dtype):
    from cellm_b200 import ops
    table = torch.randn(777, 100, device=DEV).to(dtype)
    ids = torch.tensor([0, 776, 5, 5, 300], dtype=torch.int32, device=DEV)
    e = err_word()
    out = ops.embed(table, ids, e)
    assert out.dtype == torch.float32 and torch.equal(out, table[ids.long()].float()) and e.item() == 0
    out = ops.embed(table, torch.tensor([3, 777], dtype=torch.int32, device=DEV), e)
    assert e.item() == 1 and float(out[1].abs().max()) == 0.0          # the bad id is flagged, not read


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("H", [100, 2048, 3000])
def test_add_rmsnorm(dtype, H):
    from cellm_b200 import ops
    T = 7
    x = torch.randn(T, H, device=DEV)
    delta = torch.randn(T, H, device=DEV).to(dtype)
    w = (torch.rand(H, device=DEV) + 0.5).to(dtype)
    x0 = x.clone()
    y = ops.add_rmsnorm(x, delta, w, 1e-3, dtype)
    s = x0.double() + delta.double()
    close(x, s, torch.float32, "stream")
    close(y, plain.rms_norm(s.cpu(), w.double().cpu(), 1e-3), dtype, "normed")
    rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
    x1 = x.clone()
    y = ops.add_rmsnorm(x, delta, w, 1e-3, dtype, rows)
    assert torch.equal(x, x1)                                           # selected rows leave the stream alone
    close(y, plain.rms_norm((x1.double() + delta.double())[rows.long()].cpu(), w.double().cpu(), 1e-3), dtype, "rows")
    close(ops.add_rmsnorm(x, None, w.float(), 1e-6, dtype), plain.rms_norm(x1.double().cpu(), w.double().cpu(), 1e-6), dtype, "no addend, 32-bit weight")


@pytest.mark.parametrize("dtype", DT)
def test_swiglu_and_residual_add(dtype):
    from cellm_b200 import ops
    gu = (torch.randn(5, 600, device=DEV) * 3).to(dtype)
    g, u = gu[:, :300].double(), gu[:, 300:].double()
    close(ops.swiglu(gu), g * torch.sigmoid(g) * u, dtype)
    x = torch.randn(5, 77, device=DEV)
    d = torch.randn(5, 77, device=DEV).to(dtype)
    ref = x.double() + d.double()
    ops.residual_add(x, d)
    close(x, ref, torch.float32)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("walk", [False, True])
@pytest.mark.parametrize("taps,bias", [(1, False), (2, True), (3, False), (5, True)])
def test_short_conv_portions_carry_the_state(dtype, taps, bias, walk):
    """Three requests fed in portions of 1, 2, 3 and 7 tokens, two of them in
    the same launch, against the whole-sequence convolution."""
    from cellm_b200 import ops
    H, slots = 50, 4
    lens = {0: 13, 1: 9, 2: 4}
    bcx = {r: torch.randn(n, 3 * H, device=DEV).to(dtype) for r, n in lens.items()}
    w = (torch.randn(H, taps, device=DEV) * 0.5).to(dtype)
    b = (torch.randn(H, device=DEV) * 0.5).to(dtype) if bias else None

    def whole(x):
        x = x.double().cpu()
        B, C, xt = x[:, :H], x[:, H:2 * H], x[:, 2 * H:]
        hist = torch.cat([torch.zeros(taps - 1, H, dtype=torch.float64), B * xt])
        conv = sum(hist[k:k + x.shape[0]] * w.double().cpu()[:, k] for k in range(taps))
        return C * (conv + (b.double().cpu() if bias else 0))
    state = torch.zeros(slots, max(taps - 1, 0), H, device=DEV)
    state[3] = 7.0                                    # a slot nobody uses must stay as it is
    slot_of = {0: 2, 1: 0, 2: 1}
    fed = {r: 0 for r in lens}
    got = {r: [] for r in lens}
    e = err_word()
    schedule = [[(0, 1), (1, 2)], [(0, 2), (2, 3)], [(1, 7)], [(0, 3), (2, 1)], [(0, 7)]]
    # walk: steps whose portions are all short take the one-launch kernel, as the engine would ask
    for step in schedule:
        rows = torch.cat([bcx[r][fed[r]:fed[r] + n] for r, n in step])
        cu = torch.tensor(np.cumsum([0] + [n for _, n in step]), dtype=torch.int32, device=DEV)
        seq = torch.cat([torch.full((n,), i) for i, (_, n) in enumerate(step)]).int().to(DEV)
        sl = torch.tensor([slot_of[r] for r, _ in step], dtype=torch.int32, device=DEV)
        y = ops.short_conv(rows, w, b, state, sl, seq, cu, e, max(n for _, n in step) if walk else 0)
        o = 0
        for r, n in step:
            got[r].append(y[o:o + n])
            fed[r] += n
            o += n
    assert e.item() == 0 and fed == lens and bool((state[3] == 7).all())
    for r in lens:
        close(torch.cat(got[r]), whole(bcx[r]), dtype, f"request {r}")


@pytest.mark.parametrize("taps,bias", [(2, False), (3, True), (4, False), (5, True)])
def test_short_conv_long_portions_of_several_requests(taps, bias):
    """Portions of hundreds of bfloat16 tokens (the kernel that walks runs of eight
    tokens per thread): three requests whose portions start and end off the runs'
    edges, one of them continuing from a state, and a second step that continues all."""
    from cellm_b200 import ops
    H, slots = 264, 5
    lens = {0: 530, 1: 301, 2: 95}
    g = torch.Generator(device=DEV).manual_seed(taps)
    bcx = {r: torch.randn(n, 3 * H, device=DEV, generator=g).bfloat16() for r, n in lens.items()}
    w = (torch.randn(H, taps, device=DEV, generator=g) * 0.5).bfloat16()
    b = (torch.randn(H, device=DEV, generator=g) * 0.5).bfloat16() if bias else None

    def whole(x):
        x = x.double().cpu()
        B, C, xt = x[:, :H], x[:, H:2 * H], x[:, 2 * H:]
        hist = torch.cat([torch.zeros(taps - 1, H, dtype=torch.float64), B * xt])
        conv = sum(hist[k:k + x.shape[0]] * w.double().cpu()[:, k] for k in range(taps))
        return C * (conv + (b.double().cpu() if bias else 0))
    state = torch.zeros(slots, taps - 1, H, device=DEV)
    state[4] = 7.0
    slot_of = {0: 3, 1: 0, 2: 2}
    fed = {r: 0 for r in lens}
    got = {r: [] for r in lens}
    e = err_word()
    for step in ([(0, 3)], [(0, 261), (1, 300), (2, 95)], [(1, 1), (0, 266)]):     # the first step leaves request 0 a state
        rows = torch.cat([bcx[r][fed[r]:fed[r] + n] for r, n in step])
        cu = torch.tensor(np.cumsum([0] + [n for _, n in step]), dtype=torch.int32, device=DEV)
        seq = torch.cat([torch.full((n,), i) for i, (_, n) in enumerate(step)]).int().to(DEV)
        sl = torch.tensor([slot_of[r] for r, _ in step], dtype=torch.int32, device=DEV)
        y = ops.short_conv(rows, w, b, state, sl, seq, cu, e, max(n for _, n in step))
        o = 0
        for r, n in step:
            got[r].append(y[o:o + n])
            fed[r] += n
            o += n
    assert e.item() == 0 and fed == lens and bool((state[4] == 7).all())
    for r in lens:
        close(torch.cat(got[r]), whole(bcx[r]), torch.bfloat16, f"request {r}")


@pytest.mark.parametrize("H,K,taps,bias,M", [(2048, 2048, 3, False, 8), (96, 96, 4, True, 3), (100 * 8, 64, 2, True, 33),
                                             (42, 200, 1, False, 1), (520, 1032, 3, True, 64), (2048, 2048, 3, False, 1)])
def test_in_proj_with_the_convolution_in_its_epilogue(H, K, taps, bias, M):
    """Decode steps: in_proj and the gated convolution as one kernel against the same arithmetic in 64-bit torch
    (B, C and x rounded to bfloat16 as a product would store them), four steps in a row (the state is carried in
    slots that change place from step to step), widths that do and do not fill the tiles of 42 channels; and
    against the product followed by short_conv, which it replaces."""
    from cellm_b200 import ops
    from cellm_b200.ops import gemm_bf16 as tc
    g = torch.Generator(device=DEV).manual_seed(H + taps)
    w_in = (torch.randn(3 * H, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    w = (torch.randn(H, taps, device=DEV, generator=g) * 0.5).bfloat16()
    b = (torch.randn(H, device=DEV, generator=g) * 0.5).bfloat16() if bias else None
    tiled = tc.tile_in_proj_for_conv(w_in)
    slots = M + 2
    state_a = torch.randn(slots, taps - 1, H, device=DEV, generator=g)
    state_b = state_a.clone()
    e = err_word()
    plan = tc.gemm_conv_plan(M, H, K, DEV)
    assert plan is not None
    cu = torch.arange(M + 1, dtype=torch.int32, device=DEV)
    seq = torch.arange(M, dtype=torch.int32, device=DEV)
    for step in range(4):
        x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
        sl = ((torch.arange(M, device=DEV) + step) % slots).int()
        before = state_b.double().clone()
        ref = ops.short_conv(ops.gemm(x, w_in, torch.bfloat16), w, b, state_a, sl, seq, cu, e, 1)
        got = tc.gemm_conv_bf16(x, tiled, H, w, b, state_b, sl, plan, e)
        assert e.item() == 0
        # 64-bit torch on the state the kernel started from
        bcx = bf16r(x.double() @ w_in.double().T)
        B, C, xx = bcx[:, :H], bcx[:, H:2 * H], bcx[:, 2 * H:]
        hist = torch.cat([before[sl.long()], (B * xx)[:, None, :]], dim=1)          # [M, taps, H]
        conv = (hist * w.double().T[None]).sum(dim=1)
        if bias:
            conv = conv + b.double()[None]
        close(got, C * conv, torch.bfloat16, f"step {step} against 64-bit torch")
        want_state = before.clone()
        want_state[sl.long()] = hist[:, 1:]
        close(state_b, want_state, torch.bfloat16, f"state after step {step}")        # B*x of sums rounded to bfloat16
        # the same sums rounded at the same places (the K split may differ, hence a unit of bfloat16 rounding here and there)
        close(got, ref.double().cpu(), torch.bfloat16, f"step {step} against product + short_conv")
        assert torch.allclose(state_a, state_b, rtol=2e-2, atol=1e-3)
    # a slot outside the pool is reported, and nothing is written for it
    bad = torch.full((M,), slots, dtype=torch.int32, device=DEV)
    tc.gemm_conv_bf16(torch.randn(M, K, device=DEV).bfloat16(), tiled, H, w, b, state_b, bad, plan, e)
    assert e.item() == 4
    e.zero_()


def bf16r(t):
    """Rounded to bfloat16 and back, as a product that stores its result in bfloat16 leaves it."""
    return t.to(torch.bfloat16).double()


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("hd,rot,inter", [(16, 16, False), (48, 32, False), (64, 64, True), (32, 0, False)])
def test_qk_norm_rope_and_page_write(dtype, hd, rot, inter):
    from cellm_b200 import ops
    nh, nkv, ps, pages = 6, 2, 8, 9
    pos = torch.tensor([0, 1, 17, 30, 31, 5], dtype=torch.int32, device=DEV)
    seq = torch.tensor([0, 0, 1, 1, 1, 2], dtype=torch.int32, device=DEV)
    bt = torch.tensor([[3, -1, -1, -1], [0, 8, 2, 5], [7, -1, -1, -1]], dtype=torch.int32, device=DEV)
    T = pos.numel()
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).to(dtype)
    qw, kw = (torch.rand(hd, device=DEV) + 0.5).to(dtype), (torch.rand(hd, device=DEV) + 0.5).to(dtype)
    theta = 1e4
    from cellm_b200.parts.rope import split_inv_freq
    inv = (theta ** (-(2.0 * torch.arange(rot // 2, dtype=torch.float64)) / max(rot, 1))) if rot else None
    inv_dev = split_inv_freq(theta, rot).to(DEV) if rot else None
    kp = torch.zeros(pages, nkv, ps, hd, device=DEV, dtype=dtype)
    vp = torch.zeros_like(kp)
    e = err_word()
    q = ops.qk_norm_rope(qkv, qw, kw, 1e-5, pos, seq, bt, kp, vp, ps, nh, nkv, hd, rot, inter, inv_dev, e)
    assert e.item() == 0

    def ref_heads(x, w, n):
        x = plain.rms_norm(x.double().cpu().reshape(T, n, hd), w.double().cpu(), 1e-5)
        if rot:
            if inter:     # pairs (2i, 2i+1)  (crates/cellm-kernels/src/cpu_kernels.rs:279-292)
                xr = x[..., :rot].reshape(T, n, rot // 2, 2)
                ang = pos.double().cpu()[:, None] * inv[None, :]
                c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
                r = torch.stack([xr[..., 0] * c - xr[..., 1] * s_, xr[..., 1] * c + xr[..., 0] * s_], -1).reshape(T, n, rot)
            else:
                r = plain.rope_rotate_half(x[..., :rot], pos.cpu(), theta)
            x = torch.cat([r, x[..., rot:]], -1)
        return x
    close(q.reshape(T, nh, hd), ref_heads(qkv[:, :nh * hd], qw, nh), dtype, "q")
    k_ref = ref_heads(qkv[:, nh * hd:(nh + nkv) * hd], kw, nkv)
    v_ref = qkv[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
    written = torch.zeros(pages, ps, dtype=torch.bool)
    for t in range(T):
        page, off = int(bt[seq[t], pos[t] // ps]), int(pos[t]) % ps
        close(kp[page, :, off], k_ref[t], dtype, f"k of token {t}")
        assert torch.equal(vp[page, :, off], v_ref[t])
        written[page, off] = True
    assert float(kp.float().abs().sum(dim=(1, 3)).cpu()[~written].max()) == 0.0     # nothing else was touched
    bad = bt.clone()
    bad[2, 0] = pages
    ops.qk_norm_rope(qkv, qw, kw, 1e-5, pos, seq, bad, kp, vp, ps, nh, nkv, hd, rot, inter, inv_dev, e)
    assert e.item() == 2


@pytest.mark.parametrize("nh,nkv,K,M,ps,theta", [(32, 8, 2048, 8, 16, 1e6), (3, 1, 96, 5, 8, 1e4), (4, 4, 264, 33, 32, 5e4),
                                                 (16, 2, 1024, 64, 16, 1e6), (32, 8, 2048, 1, 16, 1e6)])
def test_qkv_product_with_norm_rotation_and_cache_write_in_its_epilogue(nh, nkv, K, M, ps, theta):
    """Decode steps: the q/k/v product, the heads' norm, the rotation and the write into the pages as
    one kernel against the product followed by qk_norm_rope: one token of M requests at positions
    near and far, pages in scrambled order, an odd number of heads (a tile with a single head)."""
    from cellm_b200 import ops
    from cellm_b200.ops import gemm_bf16 as tc
    from cellm_b200.parts.rope import split_inv_freq
    hd = 64
    g = torch.Generator(device=DEV).manual_seed(nh * 100 + M)
    w = (torch.randn((nh + 2 * nkv) * hd, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    qw = (torch.rand(hd, device=DEV, generator=g) + 0.5).bfloat16()
    kw = (torch.rand(hd, device=DEV, generator=g) + 0.5).bfloat16()
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    width = 40
    pos = torch.randint(0, width * ps, (M,), device=DEV, generator=g).int()
    pos[0] = 0
    pos[-1] = width * ps - 1
    pages = M * width
    bt = torch.randperm(pages, device=DEV, generator=g).int().reshape(M, width).contiguous()
    seq = torch.arange(M, dtype=torch.int32, device=DEV)
    inv = split_inv_freq(theta, hd).to(DEV)
    kp_a = torch.zeros(pages, nkv, ps, hd, device=DEV, dtype=torch.bfloat16)
    vp_a, kp_b, vp_b = torch.zeros_like(kp_a), torch.zeros_like(kp_a), torch.zeros_like(kp_a)
    e = err_word()
    ref = ops.qk_norm_rope(ops.gemm(x, w, torch.bfloat16), qw, kw, 1e-5, pos, seq, bt, kp_a, vp_a, ps, nh, nkv, hd, hd, False, inv, e)
    plan = tc.gemm_rope_plan(M, nh, nkv, hd, K, DEV)
    assert plan is not None
    got = tc.gemm_rope_bf16(x, w, qw, kw, 1e-5, pos, bt, kp_b, vp_b, nh, nkv, inv, plan, e)
    assert e.item() == 0
    # against 64-bit torch: the plain implementation's norm and rotation on the sums rounded to bfloat16
    qkv = bf16r(x.double() @ w.double().T).cpu()
    q64 = plain.rope_rotate_half(plain.rms_norm(qkv[:, :nh * hd].reshape(M, nh, hd), qw.double().cpu(), 1e-5), pos.cpu(), theta)
    k64 = plain.rope_rotate_half(plain.rms_norm(qkv[:, nh * hd:(nh + nkv) * hd].reshape(M, nkv, hd), kw.double().cpu(), 1e-5), pos.cpu(), theta)
    v64 = qkv[:, (nh + nkv) * hd:].reshape(M, nkv, hd)
    close(got, q64.reshape(M, nh * hd), torch.bfloat16, "q against 64-bit torch")
    for t in range(M):
        page, off = int(bt[t, pos[t] // ps]), int(pos[t]) % ps
        close(kp_b[page, :, off], k64[t], torch.bfloat16, f"k of token {t} against 64-bit torch")
        close(vp_b[page, :, off], v64[t], torch.bfloat16, f"v of token {t} against 64-bit torch")
    # the same sums rounded at the same places (the K split may differ, hence a unit of bfloat16 rounding here and there)
    close(got, ref, torch.bfloat16, "q")
    close(kp_b, kp_a, torch.bfloat16, "keys")
    close(vp_b, vp_a, torch.bfloat16, "values")
    assert torch.equal(kp_b.float().abs().sum(-1) > 0, kp_a.float().abs().sum(-1) > 0)      # the same places were written
    bad = bt.clone()
    bad[M - 1, int(pos[M - 1]) // ps] = pages
    tc.gemm_rope_bf16(x, w, qw, kw, 1e-5, pos, bad, kp_b, vp_b, nh, nkv, inv, plan, e)
    assert e.item() == 2
    e.zero_()


@pytest.mark.parametrize("wdt", [torch.bfloat16, torch.float32])
def test_qk_norm_rope_long_batches_of_64_wide_heads(wdt):
    """300 tokens of 64-wide heads take the one-warp-per-token form; it must agree
    with the general kernel's result on the same rows (forced by feeding them in
    pieces shorter than 256)."""
    from cellm_b200 import ops
    from cellm_b200.parts.rope import split_inv_freq
    nh, nkv, hd, ps, T = 6, 2, 64, 16, 300
    pos = torch.arange(T, dtype=torch.int32, device=DEV) + 5
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    pages = (T + 5 + ps - 1) // ps
    bt = torch.randperm(pages).int().reshape(1, -1).to(DEV)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).bfloat16()
    qw, kw = (torch.rand(hd, device=DEV) + 0.5).to(wdt), (torch.rand(hd, device=DEV) + 0.5).to(wdt)
    inv = split_inv_freq(1e6, hd).to(DEV)
    outs = []
    for pieces in ([slice(0, T)], [slice(0, 100), slice(100, 200), slice(200, T)]):
        kp = torch.zeros(pages, nkv, ps, hd, device=DEV, dtype=torch.bfloat16)
        vp = torch.zeros_like(kp)
        e = err_word()
        q = torch.cat([ops.qk_norm_rope(qkv[sl], qw, kw, 1e-5, pos[sl], seq[sl], bt, kp, vp, ps, nh, nkv, hd, hd, False, inv, e) for sl in pieces])
        assert e.item() == 0
        outs.append((q, kp, vp))
    for a, b in zip(outs[0], outs[1]):
        assert float((a.float() - b.float()).abs().max()) <= 2 ** -7 * float(b.float().abs().max())     # one bfloat16 step


def test_rotation_angles_stay_exact_far_out():
    """At positions in the hundreds of thousands a float angle is off by whole
    hundredths of a radian; the kernel's split arithmetic is not."""
    from cellm_b200 import ops
    from cellm_b200.parts.rope import split_inv_freq
    hd, theta = 64, 1e6
    pos = torch.tensor([0, 1, 4097, 131071, 500000, 1048575], dtype=torch.int32, device=DEV)
    T = pos.numel()
    q = torch.randn(T, hd, device=DEV)
    out = ops.qk_norm_rope(q, None, None, 0.0, pos, torch.zeros(T, dtype=torch.int32, device=DEV), None, None, None, 16,
                           1, 0, hd, hd, False, split_inv_freq(theta, hd).to(DEV), err_word())
    ref = plain.rope_rotate_half(q.double().cpu().reshape(T, 1, hd), pos.cpu(), theta).reshape(T, hd)
    assert float((out.double().cpu() - ref).abs().max()) < 3e-6 * float(q.abs().max())


def paged_case(q_lens, ctx_lens, nh, nkv, hd, ps, dtype, seed=0, scale_one=None):
    g = torch.Generator().manual_seed(seed)
    totals = [c + n for c, n in zip(ctx_lens, q_lens)]
    nblk = [-(-t // ps) for t in totals]
    pages = sum(nblk) + 2
    perm = torch.randperm(pages, generator=g).tolist()
    bt = torch.full((len(q_lens), max(nblk)), -1, dtype=torch.int32)
    k_seq, v_seq, o = [], [], 0
    kp = torch.zeros(pages, nkv, ps, hd)
    vp = torch.zeros(pages, nkv, ps, hd)
    for b, t in enumerate(totals):
        bt[b, :nblk[b]] = torch.tensor(perm[o:o + nblk[b]], dtype=torch.int32)
        o += nblk[b]
        k = torch.randn(t, nkv, hd, generator=g)
        v = torch.randn(t, nkv, hd, generator=g)
        if scale_one is not None and b == scale_one[0]:
            k[scale_one[1]] *= scale_one[2]
        k, v = k.to(dtype).float(), v.to(dtype).float()
        k_seq.append(k), v_seq.append(v)
        for j in range(t):
            kp[bt[b, j // ps], :, j % ps] = k[j]
            vp[bt[b, j // ps], :, j % ps] = v[j]
    q = torch.randn(sum(q_lens), nh * hd, generator=g).to(dtype)
    return dict(q=q.to(DEV), kp=kp.to(dtype).to(DEV), vp=vp.to(dtype).to(DEV), bt=bt.to(DEV), k_seq=k_seq, v_seq=v_seq,
                q_lens=q_lens, ctx_lens=ctx_lens,
                pos=torch.cat([torch.arange(c, c + n) for c, n in zip(ctx_lens, q_lens)]).int().to(DEV),
                seq=torch.cat([torch.full((n,), b) for b, n in enumerate(q_lens)]).int().to(DEV),
                cu=torch.tensor(np.cumsum([0] + q_lens), dtype=torch.int32, device=DEV),
                ctx=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV))


def attention_reference(c, nh, nkv, hd, scale, window):
    out, o = [], 0
    for b, (n, ctx) in enumerate(zip(c["q_lens"], c["ctx_lens"])):
        q = c["q"][o:o + n].double().cpu().reshape(n, nh, hd)
        k, v = c["k_seq"][b].double(), c["v_seq"][b].double()
        res = torch.zeros(n, nh, hd, dtype=torch.float64)
        for i in range(n):
            p = ctx + i
            lo = max(0, p - window + 1) if window else 0
            for h in range(nh):
                s = (k[lo:p + 1, h // (nh // nkv)] @ q[i, h]) * scale
                res[i, h] = torch.softmax(s, 0) @ v[lo:p + 1, h // (nh // nkv)]
        out.append(res.reshape(n, nh * hd))
        o += n
    return torch.cat(out)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(4, 2, 16, 8, 0), (3, 1, 48, 16, 0), (6, 6, 80, 4, 0), (4, 2, 32, 8, 21)])
def test_attention_plain(dtype, nh, nkv, hd, ps, window):
    from cellm_b200 import ops
    c = paged_case([9, 1, 40], [0, 150, 130], nh, nkv, hd, ps, dtype, seed=1)
    e = err_word()
    out = ops.attention_plain(c["q"], c["kp"], c["vp"], c["pos"], c["seq"], c["bt"], nh, hd ** -0.5, window, e)
    assert e.item() == 0
    close(out, attention_reference(c, nh, nkv, hd, hd ** -0.5, window), dtype)


@pytest.mark.parametrize("kernel", ["plain32", "plain16", "flash", "decode", "tc"])
def test_a_far_key_among_hundreds_is_found(kernel):
    """One early key is scaled so that its score towers over 600 others: the
    output must be that key's value. A kernel that skips a page, stops short or
    reads a neighbour's page cannot pass."""
    from cellm_b200 import ops
    from cellm_b200.ops.attention import attention_decode, attention_flash, attention_tc
    dtype = torch.float32 if kernel == "plain32" else torch.bfloat16
    nh, nkv, hd, ps = 4, 2, 64, 16
    for far in (0, 15, 16, 337):                       # a page's first and last slot, and the middle of nowhere
        c = paged_case([1, 3], [640, 600], nh, nkv, hd, ps, dtype, seed=far, scale_one=(0, far, 1.0))
        kh = c["k_seq"][0][far, 0]
        c["q"][0, :hd] = (kh / kh.norm() * 60).to(dtype).to(DEV)          # head 0 of request 0 looks at key `far`
        e = err_word()
        if kernel == "flash":
            out = attention_flash(c["q"], c["kp"], c["vp"], c["cu"], c["ctx"], c["bt"], c["q_lens"], nh, 1.0, 0, e, nsplit=3)
        elif kernel == "decode":
            out = attention_decode(c["q"], c["kp"], c["vp"], c["cu"], c["ctx"], c["bt"], 2, nh, 1.0, 0, e, nsplit=3)
        elif kernel == "tc":
            out = attention_tc(c["q"], c["kp"], c["vp"], c["cu"], c["ctx"], c["bt"], c["q_lens"], nh, 1.0, 0, e)
        else:
            out = ops.attention_plain(c["q"], c["kp"], c["vp"], c["pos"], c["seq"], c["bt"], nh, 1.0, 0, e)
        assert e.item() == 0
        close(out[0, :hd], c["v_seq"][0][far, 0], dtype, f"far key {far}")
        close(out, attention_reference(c, nh, nkv, hd, 1.0, 0), dtype, f"far key {far}, all rows")


@pytest.mark.parametrize("pieces", [8, 11, 16, 24])
def test_a_far_key_among_thousands_through_every_way_the_decode_pieces_meet(pieces):
    """2,500 keys cut into 8 pieces (one cluster), 11 (a piece per CTA through the workspace), 16 and 24 (clusters of
    eight, a piece per cluster through the workspace); the towering key lies in the first piece, in a middle one (the
    second cluster's where there are two) and in the last. A merge that loses a cluster's piece, or a piece of a
    cluster, cannot pass; neither can one that keeps a stale piece of the call before (every call has another key)."""
    from cellm_b200.ops.attention import attention_decode
    nh, nkv, hd, ps = 4, 2, 64, 16
    e = err_word()
    for far in (7, 1290, 2499):
        c = paged_case([1, 1], [2500, 70], nh, nkv, hd, ps, torch.bfloat16, seed=far, scale_one=(0, far, 1.0))
        kh = c["k_seq"][0][far, 0]
        c["q"][0, :hd] = (kh / kh.norm() * 60).to(torch.bfloat16).to(DEV)
        out = attention_decode(c["q"], c["kp"], c["vp"], c["cu"], c["ctx"], c["bt"], 2, nh, 1.0, 0, e, pieces)
        close(out[0, :hd], c["v_seq"][0][far, 0], torch.bfloat16, f"{pieces} pieces, far key {far}")
        close(out, attention_reference(c, nh, nkv, hd, 1.0, 0), torch.bfloat16, f"{pieces} pieces, far key {far}, all rows")
    assert e.item() == 0


@pytest.mark.parametrize("hd,ps,nh,nkv", [(32, 8, 3, 1), (64, 16, 8, 2), (128, 32, 4, 4), (64, 4, 32, 8)])
@pytest.mark.parametrize("window", [0, 33])
def test_attention_flash(hd, ps, nh, nkv, window):
    from cellm_b200.ops.attention import attention_flash
    c = paged_case([70, 1, 5, 1], [0, 200, 59, 64], nh, nkv, hd, ps, torch.bfloat16, seed=2)
    ref = attention_reference(c, nh, nkv, hd, hd ** -0.5, window)
    e = err_word()
    for nsplit, wide in ((1, None), (3, True)):
        out = attention_flash(c["q"], c["kp"], c["vp"], c["cu"], c["ctx"], c["bt"], c["q_lens"], nh, hd ** -0.5, window, e, nsplit, wide)
        close(out, ref, torch.bfloat16, f"nsplit {nsplit}")
    d = paged_case([1, 1, 1], [3, 700, 64], nh, nkv, hd, ps, torch.bfloat16, seed=3)         # decode shape, narrow tiles
    out = attention_flash(d["q"], d["kp"], d["vp"], d["cu"], d["ctx"], d["bt"], d["q_lens"], nh, hd ** -0.5, window, e, 4, False)
    close(out, attention_reference(d, nh, nkv, hd, hd ** -0.5, window), torch.bfloat16, "decode")
    assert e.item() == 0


@pytest.mark.parametrize("ps,nh,nkv", [(16, 8, 2), (8, 2, 2), (32, 16, 1), (128, 32, 8), (64, 3, 3)])
@pytest.mark.parametrize("window", [0, 33, 300])
def test_attention_tc(ps, nh, nkv, window):
    """The tcgen05 prompt kernel: portions that end inside a tile, start after a
    context, span several key blocks; single tokens beside them; a window that
    skips whole blocks. With scale 1 the scores spread so far that the lazy
    rescaling of the accumulator runs."""
    from cellm_b200.ops.attention import attention_tc, attention_tc_supports
    hd = 64
    assert attention_tc_supports(hd, nh, nkv, ps)
    c = paged_case([300, 1, 33, 129], [0, 500, 59, 640], nh, nkv, hd, ps, torch.bfloat16, seed=6)
    e = err_word()
    for scale in (hd ** -0.5, 1.0):
        for _ in range(2):
            out = attention_tc(c["q"], c["kp"], c["vp"], c["cu"], c["ctx"], c["bt"], c["q_lens"], nh, scale, window, e)
            close(out, attention_reference(c, nh, nkv, hd, scale, window), torch.bfloat16, f"scale {scale}")
    assert e.item() == 0


def test_attention_tc_refuses_what_it_does_not_take():
    from cellm_b200.ops.attention import attention_tc, attention_tc_supports
    assert not attention_tc_supports(128, 4, 4, 16) and not attention_tc_supports(64, 6, 2, 16)
    assert not attention_tc_supports(64, 4, 2, 4) and not attention_tc_supports(64, 4, 2, 24)
    c = paged_case([40], [0], 6, 2, 64, 16, torch.bfloat16, seed=1)
    with pytest.raises(ValueError):
        attention_tc(c["q"], c["kp"], c["vp"], c["cu"], c["ctx"], c["bt"], c["q_lens"], 6, 0.125, 0, err_word())


@pytest.mark.parametrize("hd,ps,nh,nkv", [(32, 8, 3, 1), (64, 16, 8, 2), (128, 32, 4, 4), (64, 4, 32, 8), (64, 16, 16, 1)])
@pytest.mark.parametrize("window", [0, 33])
def test_attention_decode(hd, ps, nh, nkv, window):
    """Decoded tokens (and portions of two or three where the group is small)
    through the kernel with a ring per warp: unsplit, split over the CTAs of a cluster (up to 8 pieces), split
    into more pieces than a cluster holds (11: a piece per CTA through the workspace and the counters; 16: two
    clusters of eight, a piece per cluster through the workspace)."""
    from cellm_b200.ops.attention import attention_decode
    G = nh // nkv
    few = max(1, min(3, 16 // G))
    c = paged_case([1, few, 1, 1, 1], [3, 700, 64, 255, 1000], nh, nkv, hd, ps, torch.bfloat16, seed=5)
    ref = attention_reference(c, nh, nkv, hd, hd ** -0.5, window)
    e = err_word()
    for nsplit in (1, 2, 5, 8, 11, 16):
        for _ in range(2):            # twice: the counters must be back at zero
            out = attention_decode(c["q"], c["kp"], c["vp"], c["cu"], c["ctx"], c["bt"], 5, nh, hd ** -0.5, window, e, nsplit)
            close(out, ref, torch.bfloat16, f"nsplit {nsplit}")
    assert e.item() == 0


def test_window_edge():
    """The key just outside the window carries a huge score and must not count;
    the key just inside does."""
    from cellm_b200 import ops
    from cellm_b200.ops.attention import attention_flash
    nh, nkv, hd, ps, window = 2, 1, 64, 8, 24
    from cellm_b200.ops.attention import attention_decode, attention_tc
    for dtype, kernel in ((torch.float32, "plain"), (torch.bfloat16, "plain"), (torch.bfloat16, "flash"), (torch.bfloat16, "decode"),
                          (torch.bfloat16, "tc")):
        for edge, inside in ((100 - window, False), (100 - window + 1, True)):
            c = paged_case([1], [100], nh, nkv, hd, ps, dtype, seed=4)
            kh = c["k_seq"][0][edge, 0]
            c["q"][0, :hd] = (kh / kh.norm() * 50).to(dtype).to(DEV)
            e = err_word()
            if kernel == "flash":
                out = attention_flash(c["q"], c["kp"], c["vp"], c["cu"], c["ctx"], c["bt"], c["q_lens"], nh, 1.0, window, e)
            elif kernel == "decode":
                out = attention_decode(c["q"], c["kp"], c["vp"], c["cu"], c["ctx"], c["bt"], 1, nh, 1.0, window, e, 2)
            elif kernel == "tc":
                out = attention_tc(c["q"], c["kp"], c["vp"], c["cu"], c["ctx"], c["bt"], c["q_lens"], nh, 1.0, window, e)
            else:
                out = ops.attention_plain(c["q"], c["kp"], c["vp"], c["pos"], c["seq"], c["bt"], nh, 1.0, window, e)
            hit = float((out[0, :hd].float().cpu() - c["v_seq"][0][edge, 0]).abs().max()) < 0.05
            assert hit == inside, (dtype, kernel, edge)
            close(out, attention_reference(c, nh, nkv, hd, 1.0, window), dtype)


@pytest.mark.parametrize("dtype,out", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (37, 101, 53), (130, 64, 300), (5, 1000, 96)])
def test_gemm_plain(dtype, out, M, N, K):
    from cellm_b200 import ops
    a, w = torch.randn(M, K, device=DEV).to(dtype), torch.randn(N, K, device=DEV).to(dtype)
    close(ops.gemm_plain(a, w, out), a.double() @ w.double().T, out)
    big = torch.randn(M, K + 3, device=DEV).to(dtype)
    close(ops.gemm_plain(big[:, :K], w, out), big[:, :K].double() @ w.double().T, out, "strided rows")


@pytest.mark.parametrize("out", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K,bn,split", [
    (128, 128, 64, 128, 1), (200, 1000, 96, 128, 1), (300, 520, 1024, 256, 1), (100, 72, 2048, 64, 1),
    (129, 257, 72, 256, 1), (1, 1000, 224, -16, 1), (8, 512, 2048, -16, 4), (17, 130, 8192, -32, 8),
    (40, 1000, 224, -64, 1), (64, 96, 96, -64, 2), (70, 300, 4096, 64, 4),
    (130, 300, 1024, -64, 4), (500, 2048, 2048, -64, 1), (70, 520, 512, -32, 2),     # swapped tiles, several token tiles side by side
    (512, 2048, 2048, 128, 4), (300, 330, 1024, 128, 16), (200, 72, 4096, 64, 8),     # plain tiles, pieces summed by a second kernel
    (1500, 4000, 256, 256, 1), (2100, 2500, 192, 128, 1),       # more tiles than SMs: CTAs of the persistent kernel loop
    (2048, 3072, 512, 176, 1), (300, 1000, 256, 240, 1), (1300, 2048, 128, 144, 1), (200, 520, 1024, 208, 1)])   # widths between 128 and 256
def test_gemm_tcgen05(out, M, N, K, bn, split):
    from cellm_b200.ops.gemm_bf16 import error_word, gemm_tcgen05
    a = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.5).bfloat16()
    c = gemm_tcgen05(a, w, out, bn, split)
    torch.cuda.synchronize()
    assert error_word(a.device).item() == 0
    ref = a.double() @ w.double().T
    # The products of bfloat16 values are exact in 32-bit; what is left is the rounding of
    # K additions, which grows like sqrt(K) units of 32-bit rounding of the sum's size
    # (K = 2048: about 1e-4 on sums of size 40); a bfloat16 result adds one rounding to 8 bits.
    k = 2.0 ** -23 * K ** 0.5 if out == torch.float32 else 6e-3
    assert float((c.double() - ref).abs().max()) <= k * (1 + float(ref.abs().max()))


@pytest.mark.parametrize("M,ff,K,bn,split", [(8, 192, 64, -16, 1), (3, 128, 2048, -16, 4), (40, 320, 96, -64, 1), (64, 64, 512, -64, 2),
                                              (150, 256, 512, -64, 1), (100, 128, 1024, -64, 4), (400, 192, 2048, 128, 8),
                                              (130, 192, 64, 128, 1), (300, 256, 1024, 256, 1), (70, 128, 4096, 128, 4), (200, 384, 2048, 256, 2),
                                              (1300, 2560, 128, 256, 1), (2500, 1152, 64, 128, 1)])
def test_gemm_tcgen05_swiglu_epilogue(M, ff, K, bn, split):
    from cellm_b200.ops.gemm_bf16 import error_word, gemm_tcgen05
    a = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w1 = (torch.randn(ff, K, device=DEV) * K ** -0.5).bfloat16()
    w3 = (torch.randn(ff, K, device=DEV) * K ** -0.5).bfloat16()
    blocked = torch.stack([w1.reshape(ff // 64, 64, K), w3.reshape(ff // 64, 64, K)], dim=1).reshape(2 * ff, K).contiguous()
    h = gemm_tcgen05(a, blocked, torch.bfloat16, bn, split, epilogue=1)
    torch.cuda.synchronize()
    assert error_word(a.device).item() == 0 and tuple(h.shape) == (M, ff)
    g, u = a.double() @ w1.double().T, a.double() @ w3.double().T
    ref = g * torch.sigmoid(g) * u
    assert float((h.double() - ref).abs().max()) <= 6e-3 * (1 + float(ref.abs().max()))


def test_gemm_dispatch_covers_every_size():
    from cellm_b200 import ops
    for M, N, K in ((3, 50, 20), (3, 50, 24), (200, 333, 40), (64, 2048, 2048), (65, 64, 64)):
        a, w = torch.randn(M, K, device=DEV).bfloat16(), torch.randn(N, K, device=DEV).bfloat16()
        close(ops.gemm(a, w), a.double() @ w.double().T, torch.bfloat16, f"{M}x{N}x{K}")
        close(ops.gemm(a, w, torch.float32), a.double() @ w.double().T, torch.float32 if K < 64 else torch.bfloat16)
    a, w = torch.randn(9, 33, device=DEV), torch.randn(21, 33, device=DEV)
    close(ops.gemm(a, w), a.double() @ w.double().T, torch.float32)


def test_argmax_and_sampling_follow_the_plain_sampler():
    from cellm_b200 import ops
    torch.manual_seed(0)
    R, V = 6, 3001
    logits = torch.randn(R, V, device=DEV) * 3
    logits[0, 7] = logits[0, 2000] = 50.0          # equal maxima: the lower id wins
    logits[1, 5] = float("nan")
    logits[2, :] = -1.0
    assert ops.argmax(logits).tolist() == [7] + logits[1:2].nan_to_num(-1e30).argmax(-1).tolist() + [0] + logits[3:].argmax(-1).tolist()
    rng = plain.XorShift64(99)
    checked = 0
    for trial in range(40):
        temps = [0.0, 0.7, 1.3, 0.9, 0.8, 1.0]
        ks = [0, 40, 5, 0, 1024, 1]
        pens = [1.0, 1.05, 1.0, 1.3, 1.0, 2.0]
        us = [rng.next_f32() for _ in range(R)]
        recent = [[int(x) for x in torch.randint(0, V, (9,))] for _ in range(R)]
        for r in range(R):                                   # make the penalty matter: recent holds the leaders
            recent[r][:3] = logits[r].nan_to_num(-1e30).topk(3).indices.tolist()
        out = ops.sample(logits, torch.tensor(temps, device=DEV), torch.tensor(ks, dtype=torch.int32, device=DEV),
                         torch.tensor(us, device=DEV), torch.tensor(pens, device=DEV),
                         torch.tensor(recent, dtype=torch.int32, device=DEV), 1024).tolist()
        for r in range(R):
            class U:      # the plain sampler draws its own number: hand it ours
                def next_f32(self_inner):
                    return us[r]
            cands = plain.top_k_candidates(logits[r].cpu(), ks[r])
            ref = plain.select_next(cands, temps[r], pens[r], 64, recent[r], U())
            if out[r] != ref:
                # only a draw that falls within rounding of a boundary of the distribution may differ
                sc = np.array([s / pens[r] if (pens[r] > 1 and i in recent[r]) else s for i, s in cands], dtype=np.float64)
                w = np.exp((sc - sc.max()) / temps[r])
                cdf = np.cumsum(w) / w.sum()
                assert np.abs(cdf - us[r]).min() < 1e-5, (trial, r, out[r], ref)
            else:
                checked += 1
    assert checked > 200


@pytest.mark.parametrize("V", [3001, 70001])
def test_sampling_with_and_without_the_group_maxima(V):
    """The first kernel's maxima of groups of 128 logits let the second look at few logits; the choice is the
    same as one block's search of the whole row. Equal logits at the k-th place and at the top, in one group
    and across groups; a row of equal leaders in every group (more candidates than fit: the whole row is
    searched after all); a row that takes the arg-max."""
    from cellm_b200 import ops
    torch.manual_seed(V)
    R = 6
    logits = torch.randn(R, V, device=DEV) * 3
    logits[0, 7] = logits[0, V - 2] = 50.0                      # equal maxima: the lower id wins
    logits[1, 5] = float("nan")
    logits[2, ::97] = 9.0                                       # many equal leaders in every run: the lowest ids
    logits[3, 127] = logits[3, 128] = logits[3, 2048] = 40.0    # equal logits on both sides of a group's edge
    logits[4, 1000:1200] = 30.0                                 # most of the top 300 in two groups
    rng = plain.XorShift64(7)
    checked = 0
    for trial in range(30):
        temps = [0.0, 0.7, 1.3, 0.9, 0.8, 1.0]
        ks = [0, 40, 5, 3, 300, 1]
        pens = [1.0, 1.05, 1.0, 1.3, 1.0, 2.0]
        us = [rng.next_f32() for _ in range(R)]
        recent = [[int(x) for x in torch.randint(0, V, (9,))] for _ in range(R)]
        for r in range(R):
            recent[r][:3] = logits[r].nan_to_num(-1e30).topk(3).indices.tolist()
        out = ops.sample(logits, torch.tensor(temps, device=DEV), torch.tensor(ks, dtype=torch.int32, device=DEV),
                         torch.tensor(us, device=DEV), torch.tensor(pens, device=DEV),
                         torch.tensor(recent, dtype=torch.int32, device=DEV), max_top_k=300).tolist()
        one_block = ops.sample(logits, torch.tensor(temps, device=DEV), torch.tensor(ks, dtype=torch.int32, device=DEV),
                               torch.tensor(us, device=DEV), torch.tensor(pens, device=DEV),
                               torch.tensor(recent, dtype=torch.int32, device=DEV), max_top_k=300, prefilter=False).tolist()
        assert out == one_block, (trial, out, one_block)         # the same candidates in the same order
        for r in range(R):
            class U:
                def next_f32(self_inner):
                    return us[r]
            cands = plain.top_k_candidates(logits[r].cpu(), ks[r])
            ref = plain.select_next(cands, temps[r], pens[r], 64, recent[r], U())
            if out[r] != ref:
                sc = np.array([s / pens[r] if (pens[r] > 1 and i in recent[r]) else s for i, s in cands], dtype=np.float64)
                w = np.exp((sc - sc.max()) / temps[r])
                cdf = np.cumsum(w) / w.sum()
                assert np.abs(cdf - us[r]).min() < 1e-5, (trial, r, out[r], ref)
            else:
                checked += 1
    assert checked > 150
