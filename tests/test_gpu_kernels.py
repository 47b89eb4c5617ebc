"""Each kernel alone against a plain float64 reference, at sizes other than the
engine's tiny models: widths and vocabularies that are no power of two, odd head
counts and groups, head sizes in steps of 16."""
import math

import pytest
import torch

import plain_mistral as P
from braidinfer_b200.csrc.api import KernelError, get_kernels

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def K():
    return get_kernels(verbose=False)


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed + sum(shape))
    return (torch.randn(*shape, device=DEV, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(K, dtype):
    table = rnd(301, 72, dtype=dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.full((5, 72), 9.0, device=DEV)
    K.embed(table, ids, out)
    assert torch.equal(out, P.embedding(table.cpu(), ids.tolist()).to(DEV))


@pytest.mark.parametrize("width", [72, 1000, 4099])
@pytest.mark.parametrize("wd, od", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.float32, torch.bfloat16)])
def test_rmsnorm(K, width, wd, od):
    x = rnd(7, width, scale=3.0)
    w = (1 + rnd(width, scale=0.1, seed=1)).to(wd)
    out = torch.full((7, width), 9.0, device=DEV, dtype=od)
    K.rmsnorm(x, w, out, 3e-6)
    ref = P.rmsnorm(x.double().cpu(), w.double().cpu(), 3e-6)
    tol = 2e-6 if od == torch.float32 else 1 / 128
    assert ((out.double().cpu() - ref).abs() <= tol * ref.abs() + 1e-6).all()
    # gathered rows (the rows whose logits are wanted), with an absent row
    idx = torch.tensor([6, 0, -1, 3], dtype=torch.int32, device=DEV)
    out2 = torch.full((4, width), 9.0, device=DEV, dtype=od)
    K.rmsnorm(x, w, out2, 3e-6, row_index=idx)
    assert torch.equal(out2[0], out[6]) and torch.equal(out2[1], out[0]) and torch.equal(out2[3], out[3])
    assert float(out2[2].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul_and_residual_add_and_cast(K, dtype):
    gu = rnd(5, 2 * 177, dtype=dtype, scale=2.0)
    out = torch.empty(5, 177, device=DEV, dtype=dtype)
    K.silu_mul(gu, out)
    g, u = gu[:, :177].double(), gu[:, 177:].double()
    ref = g / (1 + torch.exp(-g)) * u
    tol = 1e-6 if dtype == torch.float32 else 1 / 128
    assert ((out.double() - ref).abs() <= tol * ref.abs() + 1e-6).all()
    h = rnd(5, 177)
    h0 = h.clone()
    K.residual_add(h, out)
    assert torch.equal(h, h0 + out.float())
    a = rnd(1000, dtype=torch.float32)
    b = torch.empty(1000, device=DEV, dtype=torch.bfloat16)
    K.cast(a, b)
    assert torch.equal(b, a.bfloat16())


def make_cache(n_seqs, lens, nkh, hd, dtype, shuffle_seed=0, page=64):
    need = [-(-l // page) for l in lens]
    total = sum(need) + 2
    cache = torch.zeros(total, 2, nkh, page, hd, device=DEV, dtype=dtype)
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(shuffle_seed)).tolist()
    table = torch.full((n_seqs, max(need)), -1, dtype=torch.int32)
    k = 0
    for i, n in enumerate(need):
        for c in range(n):
            table[i, c] = perm[k]
            k += 1
    return cache, table.to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pairing, rope_dim", [("half", 48), ("adjacent", 48), ("half", 32)])
def test_rope_and_cache_write(K, dtype, pairing, rope_dim):
    nqh, nkh, hd, theta = 5, 3, 48, 12345.0
    seqs = [(60, 10), (0, 3)]                       # (cache length before, new tokens); the first crosses a page
    cache, table = make_cache(2, [b + n for b, n in seqs], nkh, hd, dtype)
    rows = sum(n for _, n in seqs) + 2              # two padding rows
    qkv = rnd(rows, (nqh + 2 * nkh) * hd, dtype=dtype)
    before = qkv.clone()
    pos = [p for b, n in seqs for p in range(b, b + n)] + [0, 0]
    seq = [i for i, (b, n) in enumerate(seqs) for _ in range(n)] + [-1, -1]
    inv = P.inv_freq(rope_dim, theta).to(DEV)
    K.rope_kv_write(qkv, inv, torch.tensor(pos, dtype=torch.int32, device=DEV),
                    torch.tensor(seq, dtype=torch.int32, device=DEV), table, cache, nqh, nkh, hd, rope_dim,
                    pairing == "adjacent", 64)
    K.check_device_errors()
    assert torch.equal(qkv[-2:], before[-2:])       # padding rows untouched
    tol = 1e-5 if dtype == torch.float32 else 1 / 100
    x = before[:-2].double().cpu().view(rows - 2, nqh + 2 * nkh, hd)
    p = torch.tensor(pos[:-2])
    want_q = x[:, :nqh].clone()
    want_k = x[:, nqh:nqh + nkh].clone()
    want_q[..., :rope_dim] = P.rope(x[:, :nqh, :rope_dim].contiguous(), p, theta, pairing)
    want_k[..., :rope_dim] = P.rope(x[:, nqh:nqh + nkh, :rope_dim].contiguous(), p, theta, pairing)
    got = qkv[:-2].double().cpu().view(rows - 2, nqh + 2 * nkh, hd)
    assert (got[:, :nqh] - want_q).abs().max() < tol * 4
    assert torch.equal(got[:, nqh + nkh:], x[:, nqh + nkh:])               # values are not rotated
    for r, (s, ps) in enumerate(zip(seq[:-2], pos[:-2])):
        page = int(table[s, ps // 64])
        kc = cache[page, 0, :, ps % 64].double().cpu()
        vc = cache[page, 1, :, ps % 64].double().cpu()
        assert (kc - want_k[r]).abs().max() < tol * 4
        assert torch.equal(vc, x[r, nqh + nkh:])


def attention_reference(q, k_all, v_all, pos, window):
    """q [nqh, hd] at position pos over keys/values [len, nkh, hd]: plain softmax."""
    nqh, hd = q.shape
    nkh = k_all.shape[1]
    out = torch.empty(nqh, hd, dtype=torch.float64)
    lo = max(0, pos - window + 1) if window else 0
    for h in range(nqh):
        kv = h // (nqh // nkh)
        s = (k_all[lo:pos + 1, kv] @ q[h]) / math.sqrt(hd)
        out[h] = torch.softmax(s, 0) @ v_all[lo:pos + 1, kv]
    return out


def attention_case(K, which, dtype, hd, nqh, nkh, seqs, window, n_splits=1, few=False, plant=None, spoil=None):
    """seqs: (cache length before, new tokens).  `plant` = (seq, query offset, key position):
    that key is made to dominate that query's scores, its value made distinctive.
    `spoil` = (seq, block, value): that entry of the page table is overwritten before the launch."""
    lens = [b + n for b, n in seqs]
    cache, table = make_cache(len(seqs), lens, nkh, hd, dtype, shuffle_seed=3)
    kv_ref = []
    for i, L in enumerate(lens):
        k = rnd(L, nkh, hd, dtype=dtype, seed=10 + i)
        v = rnd(L, nkh, hd, dtype=dtype, seed=20 + i)
        kv_ref.append((k, v))
    rows = sum(n for _, n in seqs)
    W = (nqh + 2 * nkh) * hd
    qkv = rnd(rows + 1, W, dtype=dtype, seed=5)
    q_start, r = [], 0
    for b, n in seqs:
        q_start.append(r)
        r += n
    if plant is not None:
        s, qo, kp = plant
        row = q_start[s] + qo
        k, v = kv_ref[s]
        qv = qkv[row, :nqh * hd].view(nqh, hd)
        g = nqh // nkh
        for h in range(nqh):
            qv[h] = qv[(h // g) * g]                                    # the heads of a group ask alike
            k[kp, h // g] = (qv[h].float() * 3.0).to(dtype)             # q . k is large and positive
        v[kp] = 5.0
    for i, (k, v) in enumerate(kv_ref):
        for p_ in range(lens[i]):
            page = int(table[i, p_ // 64])
            cache[page, 0, :, p_ % 64] = k[p_]
            cache[page, 1, :, p_ % 64] = v[p_]
    if spoil is not None:
        table[spoil[0], spoil[1]] = spoil[2]
    pos = [p_ for b, n in seqs for p_ in range(b, b + n)] + [0]
    seq = [i for i, (b, n) in enumerate(seqs) for _ in range(n)] + [-1]
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    out = torch.full((rows + 1, nqh * hd), 9.0, device=DEV, dtype=dtype)
    if which == "simple":
        K.attn_simple(qkv, out, cache, table, t(pos), t(seq), nqh, nkh, hd, 64, window, 1 / math.sqrt(hd))
    elif which == "tc":
        out.zero_()
        K.attn_tc(qkv, out, cache, table, t(q_start), t([n for _, n in seqs]), t([b for b, _ in seqs]),
                  len(seqs), max(n for _, n in seqs), nqh, nkh, hd, window, 1 / math.sqrt(hd))
        K.check_device_errors()
    else:
        K.attn_mma(qkv, out, cache, table, t(q_start), t([n for _, n in seqs]), t([b for b, _ in seqs]), t(seq),
                   len(seqs), max(n for _, n in seqs), nqh, nkh, hd, window, 1 / math.sqrt(hd),
                   n_splits=n_splits, few_tokens=few)
    torch.cuda.synchronize()
    worst = 0.0
    for r_ in range(rows):
        s = seq[r_]
        k, v = kv_ref[s]
        q = qkv[r_, :nqh * hd].view(nqh, hd).double().cpu()
        ref = attention_reference(q, k.double().cpu(), v.double().cpu(), pos[r_], window)
        worst = max(worst, (out[r_].view(nqh, hd).double().cpu() - ref).abs().max().item())
    return worst, out, q_start


ATTN_SHAPES = [
    # hd, nqh, nkh, seqs, window
    (16, 4, 2, [(0, 70), (5, 9), (0, 1)], None),
    (32, 6, 2, [(0, 130), (200, 3)], 8),
    (48, 5, 5, [(3, 140)], 70),
    (80, 6, 3, [(0, 65), (64, 64)], 64),
    (128, 8, 2, [(0, 300), (100, 50)], None),
    (256, 3, 1, [(0, 90)], 17),
]


@pytest.mark.parametrize("hd, nqh, nkh, seqs, window", ATTN_SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_plain_attention_kernel(K, dtype, hd, nqh, nkh, seqs, window):
    worst, _, _ = attention_case(K, "simple", dtype, hd, nqh, nkh, seqs, window)
    assert worst < (2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("hd, nqh, nkh, seqs, window", ATTN_SHAPES)
def test_tensor_core_attention_kernel(K, hd, nqh, nkh, seqs, window):
    worst, _, _ = attention_case(K, "mma", torch.bfloat16, hd, nqh, nkh, seqs, window)
    assert worst < 2e-2


@pytest.mark.parametrize("hd, nqh, nkh, seqs, window", [
    (128, 8, 2, [(0, 300), (100, 50)], None),
    (128, 32, 8, [(0, 129), (0, 1), (63, 2), (0, 64)], None),
    (128, 4, 4, [(0, 400)], 130),
    (128, 6, 2, [(5, 260), (300, 40)], 64),            # a group of 3: 126 of the 128 rows in use
    (64, 8, 2, [(0, 200), (5, 90)], None),
    (64, 5, 1, [(0, 270)], 100),
    (64, 16, 16, [(128, 128)], None),
])
def test_tcgen05_attention_kernel(K, hd, nqh, nkh, seqs, window):
    worst, _, _ = attention_case(K, "tc", torch.bfloat16, hd, nqh, nkh, seqs, window)
    assert worst < 2e-2


@pytest.mark.parametrize("hd, nqh, nkh, seqs, window, scale_q", [
    (128, 32, 8, [(0, 1500)], None, 1.0),              # 376 CTAs: more than the GPU holds at once
    (128, 32, 8, [(0, 1100), (900, 700)], 600, 4.0),   # the same with a window and a running maximum that moves
    (64, 32, 8, [(0, 2048)], None, 1.0),
])
def test_tcgen05_attention_in_more_ctas_than_run_at_once(K, hd, nqh, nkh, seqs, window, scale_q):
    """CTAs that start when others end meet a CTA in mid-flight on their SM; a barrier that the softmax
    warps could run two phases ahead of showed only then.  Compared with the mma.sync kernel, which the
    tests above hold against the float64 reference."""
    torch.manual_seed(0)
    lens = [b + n for b, n in seqs]
    cache, table = make_cache(len(seqs), lens, nkh, hd, torch.bfloat16, shuffle_seed=5)
    cache.copy_(torch.randn(cache.shape, device=DEV).to(torch.bfloat16))
    rows = sum(n for _, n in seqs)
    qkv = torch.randn(rows, (nqh + 2 * nkh) * hd, device=DEV)
    qkv[:, :nqh * hd] *= scale_q
    qkv = qkv.to(torch.bfloat16)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    q_start, seq, r = [], [], 0
    for i, (b, n) in enumerate(seqs):
        q_start.append(r)
        seq += [i] * n
        r += n
    args = (t(q_start), t([n for _, n in seqs]), t([b for b, _ in seqs]))
    ref = torch.zeros(rows, nqh * hd, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros_like(ref)
    for _ in range(3):                                   # the interleaving differs from launch to launch
        K.attn_mma(qkv, ref, cache, table, *args, t(seq), len(seqs), max(n for _, n in seqs), nqh, nkh, hd, window,
                   1 / math.sqrt(hd))
        out.zero_()
        K.attn_tc(qkv, out, cache, table, *args, len(seqs), max(n for _, n in seqs), nqh, nkh, hd, window,
                  1 / math.sqrt(hd))
        torch.cuda.synchronize()
        K.check_device_errors()
        # both are rounded to bfloat16: one unit in the last place is 2^-8 of the value
        assert ((out.float() - ref.float()).abs() / (1.0 + ref.float().abs())).max().item() < 1.5e-2


def test_tcgen05_attention_gives_the_same_bits_every_time(K):
    """Sequences of very unequal lengths in one launch: the short one's CTAs leave at once, and the
    CTAs that take their places start at odd moments beside CTAs in mid-flight.  A softmax warp that
    looked at the barrier of the second product only at the end could find it two phases behind, take
    that for done and read its output early: a whole warp's rows came out differently now and then."""
    torch.manual_seed(0)
    hd, nqh, nkh, seqs = 128, 32, 8, [(0, 500), (0, 37), (0, 260)]
    lens = [b + n for b, n in seqs]
    cache, table = make_cache(len(seqs), lens, nkh, hd, torch.bfloat16, shuffle_seed=7)
    cache.copy_(torch.randn(cache.shape, device=DEV).to(torch.bfloat16))
    rows = sum(n for _, n in seqs)
    qkv = torch.randn(rows, (nqh + 2 * nkh) * hd, device=DEV).to(torch.bfloat16)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    q_start, r = [], 0
    for b, n in seqs:
        q_start.append(r)
        r += n
    args = (t(q_start), t([n for _, n in seqs]), t([b for b, _ in seqs]))
    junk = torch.randn(1024, 1024, device=DEV)
    first = None
    for window in (None, 160):
        first = None
        for it in range(60):
            out = torch.zeros(rows, nqh * hd, device=DEV, dtype=torch.bfloat16)
            if it % 2:
                junk @ junk                                  # other work before it shifts the timing
            K.attn_tc(qkv, out, cache, table, *args, len(seqs), max(n for _, n in seqs), nqh, nkh, hd, window,
                      1 / math.sqrt(hd))
            torch.cuda.synchronize()
            if first is None:
                first = out
            else:
                assert torch.equal(out, first), f"run {it} differs from run 0 (window {window})"
    K.check_device_errors()


@pytest.mark.parametrize("hd, nqh, nkh, seqs, window, splits", [
    (128, 32, 8, [(2047, 1), (100, 1), (0, 1), (63, 1), (64, 1)], None, 8),
    (128, 32, 8, [(700, 1), (100, 1)], 128, 4),
    (32, 6, 2, [(300, 1), (5, 1)], 8, 3),
    (16, 4, 2, [(30, 3), (64, 2)], None, 2),
    (64, 40, 2, [(200, 1)], None, 5),
    (96, 7, 7, [(129, 1)], None, 1),
])
def test_tensor_core_attention_sliced_context(K, hd, nqh, nkh, seqs, window, splits):
    worst, _, _ = attention_case(K, "mma", torch.bfloat16, hd, nqh, nkh, seqs, window, n_splits=splits, few=True)
    assert worst < 2e-2


@pytest.mark.parametrize("which", ["simple", "mma", "mma_sliced", "tc"])
def test_a_far_key_among_hundreds_and_the_windows_edge(K, which):
    kw = dict(n_splits=7, few=True) if which == "mma_sliced" else {}
    name = which if which in ("simple", "tc") else "mma"
    hd, nqh, nkh = 64, 4, 2
    # a key at position 3, 700 tokens back, owns the softmax: the output is its value
    worst, out, qs = attention_case(K, name, torch.bfloat16, hd, nqh, nkh, [(703, 1)], None, plant=(0, 0, 3), **kw)
    assert worst < 3e-2 and abs(float(out[0].float().mean()) - 5.0) < 0.1
    # window 100, query at 703: position 604 is the last one inside, 603 the first one outside
    worst, out, qs = attention_case(K, name, torch.bfloat16, hd, nqh, nkh, [(703, 1)], 100, plant=(0, 0, 604), **kw)
    assert worst < 3e-2 and abs(float(out[0].float().mean()) - 5.0) < 0.1
    worst, out, qs = attention_case(K, name, torch.bfloat16, hd, nqh, nkh, [(703, 1)], 100, plant=(0, 0, 603), **kw)
    assert worst < 3e-2 and abs(float(out[0].float().mean())) < 1.0
    # the same in a prompt: query 650 of a 704-token prompt looks at key 1
    if which != "mma_sliced":
        worst, out, qs = attention_case(K, name, torch.bfloat16, hd, nqh, nkh, [(0, 704)], None, plant=(0, 650, 1))
        assert worst < 3e-2 and abs(float(out[650].float().mean()) - 5.0) < 0.1
        # and at key 640, ten tiles in: what was summed before under a small maximum has to be scaled down
        worst, out, qs = attention_case(K, name, torch.bfloat16, hd, nqh, nkh, [(0, 704)], None, plant=(0, 650, 640))
        assert worst < 3e-2 and abs(float(out[650].float().mean()) - 5.0) < 0.1


@pytest.mark.parametrize("which, dtype", [("simple", torch.float32), ("simple", torch.bfloat16), ("mma", torch.bfloat16),
                                          ("mma_sliced", torch.bfloat16), ("mma_prompt", torch.bfloat16),
                                          ("tc", torch.bfloat16)])
@pytest.mark.parametrize("bad", [-1, 10 ** 6])
def test_a_broken_page_table_raises_the_error_flag_and_is_never_followed(K, which, dtype, bad):
    """A table entry of a visible position that is absent (-1) or beyond the cache: every attention
    kernel checks the entry before it makes an address from it, reads page 0 instead and raises
    the device error flag, which the host turns into a KernelError."""
    hd, nqh, nkh = 64, 4, 2
    K.check_device_errors()
    if which in ("mma_prompt", "tc"):
        seqs, kw = [(0, 200)], {}
    else:
        seqs, kw = [(199, 1)], (dict(n_splits=3, few=True) if which == "mma_sliced" else {})
    name = which if which in ("simple", "tc") else "mma"
    attention_case(K, name, dtype, hd, nqh, nkh, seqs, None, **kw)          # the sound table: no flag
    K.check_device_errors()
    try:
        attention_case(K, name, dtype, hd, nqh, nkh, seqs, None, spoil=(0, 1, bad), **kw)
    except KernelError:
        return                                               # the tcgen05 case checks its flag itself
    with pytest.raises(KernelError, match="page"):
        K.check_device_errors()
    K.check_device_errors()                                  # the flag is cleared once it was reported


def test_plain_product_refuses_operands_of_two_element_types(K):
    """The plain product reads both operands as one element type; a float32 x with a bfloat16 w
    would read w past its end, so the call is refused on the host."""
    x, w = rnd(4, 64), rnd(32, 64, dtype=torch.bfloat16, seed=1)
    with pytest.raises(KernelError, match="one element type"):
        K.gemm_simt(x, w, torch.empty(4, 32, device=DEV))
    with pytest.raises(KernelError, match="do not fit"):
        K.gemm_simt(x, rnd(32, 48), torch.empty(4, 32, device=DEV))


@pytest.mark.parametrize("n, m, k", [(5, 70, 33), (64, 64, 64), (130, 200, 96), (1, 331, 120)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_plain_matrix_product(K, dtype, n, m, k):
    x, w = rnd(n, k, dtype=dtype), rnd(m, k, dtype=dtype, seed=1)
    ref = x.double() @ w.double().t()
    out = torch.full((n, m), 9.0, device=DEV)
    K.gemm_simt(x, w, out)
    assert (out.double() - ref).abs().max() < 1e-4 * max(1.0, ref.abs().max().item())
    res = rnd(n, m, seed=2)
    want = res.double() + ref
    K.gemm_simt(x, w, res, residual=res)
    assert (res.double() - want).abs().max() < 1e-4 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("n, m, k, sk", [
    (16, 128, 64, False), (33, 200, 96, False), (1, 331, 120, False), (300, 1000, 520, False),
    (700, 384, 1024, False), (2048, 512, 256, False), (8, 512, 4096, True), (20, 256, 2048, True),
    (64, 1408, 1024, True), (3, 200, 8200, True), (1, 128, 64, True), (40, 20000, 320, True), (300, 640, 2048, True),
    (2500, 400, 192, False), (4300, 136, 64, False),       # 10 and 17 token tiles: groups of 8 and a narrower last group
    (2500, 400, 192, True), (4300, 136, 64, True), (700, 384, 1024, True)])      # the same walk with partial sums
def test_tensor_core_matrix_product(K, n, m, k, sk):
    x, w = rnd(n, k, dtype=torch.bfloat16, scale=0.5), rnd(m, k, dtype=torch.bfloat16, scale=0.5, seed=1)
    ref = x.double() @ w.double().t()
    scale = max(1.0, ref.abs().max().item())
    out = torch.full((n, m), 9.0, device=DEV)
    K.gemm_tc(x, w, out, stream_k=sk)
    assert (out.double() - ref).abs().max() < 1e-5 * scale
    plain = torch.empty(n, m, device=DEV)
    K.gemm_simt(x, w, plain)
    assert (out - plain).abs().max() < 1e-5 * scale                  # beside its plain twin
    outb = torch.full((n, m), 9.0, device=DEV, dtype=torch.bfloat16)
    K.gemm_tc(x, w, outb, stream_k=sk)
    assert (outb.double() - ref).abs().max() < scale / 128
    res = rnd(n, m, seed=2)
    want = res.double() + ref
    K.gemm_tc(x, w, res, residual=res, stream_k=sk)
    assert (res.double() - want).abs().max() < 1e-5 * scale
    K.check_device_errors()


@pytest.mark.parametrize("n, inter, k, sk", [(300, 384, 512, False), (17, 200, 96, False), (20, 256, 2048, True),
                                             (64, 1000, 520, True), (8, 14336, 512, True), (700, 1000, 264, False),
                                             (2048, 176, 64, False), (5, 63, 128, True), (2400, 300, 128, False),
                                             (2400, 300, 128, True), (300, 1000, 264, True)])
def test_tensor_core_swiglu_epilogue(K, n, inter, k, sk):
    from braidinfer_b200.csrc.api import interleave_gate_up
    x = rnd(n, k, dtype=torch.bfloat16, scale=0.5)
    w = rnd(2 * inter, k, dtype=torch.bfloat16, scale=0.2, seed=1)
    ref = x.double() @ w.double().t()
    g, u = ref[:, :inter], ref[:, inter:]
    want = g / (1 + torch.exp(-g)) * u
    out = torch.full((n, inter), 9.0, device=DEV, dtype=torch.bfloat16)
    K.gemm_tc(x, interleave_gate_up(w[:inter], w[inter:]), out, swiglu=True, stream_k=sk)
    assert ((out.double() - want).abs() <= want.abs() / 100 + 1e-3).all()


@pytest.mark.parametrize("n, m, k", [(129, 136, 64), (300, 1000, 520), (700, 20000, 200), (2500, 400, 192),
                                     (4300, 136, 72), (256, 256, 4104), (300, 331, 520), (513, 778, 128)])
@pytest.mark.parametrize("direct_out", [False, True])
def test_product_on_pairs_of_sms(K, n, m, k, direct_out):
    """Tiles of 256 x 256 on two SMs each (more tiles than pairs at 20,000 rows; ragged edges in all three
    sizes): float64 beside it, and the bits of the one-SM kernel with the same token tile, in all three
    epilogues, with the output leaving through TMA and thread by thread (331 and 389 bfloat16 outputs a row
    cannot be addressed by TMA: those go thread by thread whatever is asked)."""
    import functools
    pair_product = functools.partial(K.gemm_tc_pair, direct_out=direct_out)
    from braidinfer_b200.csrc.api import interleave_gate_up
    x, w = rnd(n, k, dtype=torch.bfloat16, scale=0.5), rnd(m, k, dtype=torch.bfloat16, scale=0.5, seed=1)
    ref = x.double() @ w.double().t()
    scale = max(1.0, ref.abs().max().item())
    for dtype, tol in ((torch.float32, 1e-5 * scale), (torch.bfloat16, scale / 128)):
        pair, single = (torch.full((n, m), 9.0, device=DEV, dtype=dtype) for _ in range(2))
        pair_product(x, w, pair)
        K.gemm_tc(x, w, single, block_n=256)
        assert (pair.double() - ref).abs().max() < tol
        assert torch.equal(pair, single)
    res = rnd(n, m, seed=2)
    res1 = res.clone()
    pair_product(x, w, res, residual=res)
    K.gemm_tc(x, w, res1, residual=res1, block_n=256)
    assert torch.equal(res, res1)
    inter = m // 2
    wi = interleave_gate_up(w[:inter], w[inter:2 * inter])
    pair, single = (torch.full((n, inter), 9.0, device=DEV, dtype=torch.bfloat16) for _ in range(2))
    pair_product(x, wi, pair, swiglu=True)
    K.gemm_tc(x, wi, single, swiglu=True, block_n=256)
    g, u = ref[:, :inter], ref[:, inter:2 * inter]
    want = g / (1 + torch.exp(-g)) * u
    # gate and up carry the float32 product's error e <= 1e-5 * scale each (asserted above); |silu'| <= 1.1 and
    # |silu(g)| <= |g| pass it on as 1.1 e |u| + e |g|, beside the bfloat16 rounding of the result
    passed_on = 1e-5 * scale * (1.1 * u.abs() + g.abs())
    assert ((pair.double() - want).abs() <= want.abs() / 100 + passed_on + 1e-3).all()
    assert torch.equal(pair, single)
    K.check_device_errors()


def test_stream_k_refuses_a_workspace_that_is_too_small_and_takes_any_token_tile(K):
    """The partial sums of a stream-k product must fit the workspace it is given: the entry point
    checks that on the host for the very plan the kernel walks, whatever token tile is named."""
    from braidinfer_b200.csrc.api import KernelError, F32, BF16
    x, w = rnd(300, 256, dtype=torch.bfloat16), rnd(512, 256, dtype=torch.bfloat16, seed=1)
    want = x.double() @ w.double().t()
    for tile in (128, 256):                                         # 3 token tiles, or 2
        out = torch.full((300, 512), float("nan"), device=DEV, dtype=torch.bfloat16)
        K.gemm_tc(x, w, out, block_n=tile, stream_k=True)
        K.check_device_errors()
        assert (out.double() - want).abs().max().item() < want.abs().max().item() / 128      # bfloat16 output
    need = K.lib.braid_gemm_tc_workspace_bytes(300, 512, 256, 128)
    assert need > 0 and 0 < K.lib.braid_gemm_tc_workspace_bytes(300, 512, 256, 256) != need        # sized for the tile named
    assert K.lib.braid_gemm_tc_workspace_bytes(300, 512, 256, 48) == -1
    ws = torch.empty(need // 4, dtype=torch.float32, device=DEV)
    out = torch.empty(300, 512, device=DEV, dtype=torch.bfloat16)
    args = lambda nbytes, tile: (x.data_ptr(), w.data_ptr(), out.data_ptr(), None, ws.data_ptr(), nbytes, BF16, 0,
                                 300, 512, 256, 256, 256, 512, tile, 1, None, None, 0, 0, 0.0, 0.0, None,
                                 K._error_flag.data_ptr() + 4, K._stream())
    assert K.lib.braid_gemm_tc(*args(need - 4, 128)) != 0            # refused on the host: nothing is launched
    assert b"bytes of workspace" in K.lib.braid_last_error()
    assert K.lib.braid_gemm_tc(*args(need, 48)) != 0 and b"token tile" in K.lib.braid_last_error()
    assert K.lib.braid_gemm_tc(*args(need, 128)) == 0
    K.check_device_errors()
    assert (out.double() - want).abs().max().item() < want.abs().max().item() / 128


def shares_of(t, n_shares):
    """A tensor's sums of squares by row, cut into shares of unequal size (as a kernel may leave them)."""
    n, width = t.shape
    cuts = [0] + sorted(torch.randperm(width - 1, generator=torch.Generator().manual_seed(n_shares))[:n_shares - 1].add(1).tolist()) + [width]
    shares = torch.zeros(n_shares, -(-n // 4) * 4, device=DEV)
    for i in range(n_shares):
        shares[i, :n] = t[:, cuts[i]:cuts[i + 1]].double().pow(2).sum(1).float()
    return shares


@pytest.mark.parametrize("n, width, k", [(8, 4096, 1024), (3, 328, 520), (64, 1000, 256), (1, 72, 64), (20, 5120, 128),
                                         (128, 516, 192)])
def test_reduce_and_the_inputs_of_a_scaled_norm(K, n, width, k):
    """h += partial sums, bfloat16(h * w) and the shares of the rows' sums of squares, by CTAs of 512 columns:
    float64 beside it, the bits of the plain reduce for h, and the same kernel on a complete h."""
    x, wt = rnd(n, k, dtype=torch.bfloat16, scale=0.5), rnd(width, k, dtype=torch.bfloat16, scale=0.5, seed=1)
    gamma = (1 + rnd(width, seed=3, scale=0.3)).to(torch.bfloat16)
    h0 = rnd(n, width, seed=4)
    want_h = h0.double() + x.double() @ wt.double().t()
    h, hb = h0.clone(), torch.full((n, width), 9.0, device=DEV, dtype=torch.bfloat16)
    scale = K.streamk_reduce_prep(K.gemm_tc_partial(x, wt), h, gamma, hb, 1e-5)
    assert K.pending_partial is None
    big = max(1.0, want_h.abs().max().item())
    assert (h.double() - want_h).abs().max() < 1e-5 * big
    plain = h0.clone()
    K.gemm_tc(x, wt, plain, residual=plain, stream_k=True)
    assert torch.equal(h, plain)
    want_hb = h.double() * gamma.double()
    assert ((hb.double() - want_hb).abs() <= want_hb.abs() / 250 + 1e-30).all()          # one bfloat16 rounding
    want_rs = torch.rsqrt(h.double().pow(2).mean(1) + 1e-5)
    assert scale.shares.shape[0] == -(-width // 512)
    assert ((scale.values()[:n].double() - want_rs).abs() / want_rs).max() < 1e-5
    # a complete h: the same numbers without partial sums
    hb2 = torch.empty_like(hb)
    again = K.streamk_reduce_prep(None, h, gamma, hb2, 1e-5)
    assert torch.equal(hb, hb2) and torch.equal(scale.shares[:, :n], again.shares[:, :n])
    K.check_device_errors()


@pytest.mark.parametrize("n, m, k, sk", [(8, 512, 256, False), (100, 640, 512, False), (40, 328, 264, False),
                                         (8, 4096, 512, True), (20, 1408, 1024, True), (100, 640, 2048, True)])
def test_products_apply_a_row_scale(K, n, m, k, sk):
    """Whole tiles in their epilogue, stream-k products in the kernel that adds them up: store and SwiGLU."""
    from braidinfer_b200.csrc.api import RowScale, interleave_gate_up
    x, w = rnd(n, k, dtype=torch.bfloat16, scale=0.5), rnd(m, k, dtype=torch.bfloat16, scale=0.5, seed=1)
    sc = RowScale(shares_of(rnd(n, 200, seed=5, scale=2.0), 3), 200, 1e-5)
    rs = sc.values()[:n].double()[:, None]
    assert ((rs[:, 0] - torch.rsqrt(rnd(n, 200, seed=5, scale=2.0).double().pow(2).mean(1) + 1e-5)).abs() / rs[:, 0]).max() < 1e-5
    ref = (x.double() @ w.double().t()) * rs
    big = max(1.0, ref.abs().max().item())
    out = torch.empty(n, m, device=DEV)
    K.gemm_tc(x, w, out, stream_k=sk, in_scale=sc)
    assert (out.double() - ref).abs().max() < 1e-5 * big
    inter = m // 2
    g, u = ref[:, :inter], ref[:, inter:2 * inter]
    want = g / (1 + torch.exp(-g)) * u
    act = torch.empty(n, inter, device=DEV, dtype=torch.bfloat16)
    K.gemm_tc(x, interleave_gate_up(w[:inter], w[inter:2 * inter]), act, swiglu=True, stream_k=sk, in_scale=sc)
    assert ((act.double() - want).abs() <= want.abs() / 100 + 1e-5 * big * (1.1 * u.abs() + g.abs()) + 1e-3).all()
    with pytest.raises(KernelError, match="row scale"):
        K.gemm_tc(x, w, out, residual=out, stream_k=sk, in_scale=sc)
    K.pending_partial = None
    K.check_device_errors()


def test_tensor_core_product_refuses_what_tma_cannot_address(K):
    x, w = rnd(4, 100, dtype=torch.bfloat16), rnd(128, 100, dtype=torch.bfloat16)     # row stride 100 is no multiple of 8
    assert not K.gemm_tc_eligible(x, w)
    with pytest.raises(KernelError, match="multiples of 8"):
        K.gemm_tc(x, w, torch.empty(4, 128, device=DEV))
    with pytest.raises(KernelError, match="multiples of 8"):
        K.gemm_tc_pair(x, w, torch.empty(4, 128, device=DEV))
    x8, w8 = rnd(4, 64, dtype=torch.bfloat16), rnd(128, 64, dtype=torch.bfloat16)
    with pytest.raises(KernelError, match="residual epilogue"):
        K.gemm_tc_pair(x8, w8, torch.empty(4, 128, device=DEV, dtype=torch.bfloat16),
                       residual=torch.empty(4, 128, device=DEV))
    with pytest.raises(KernelError, match="interleaved weight rows"):
        K.gemm_tc_pair(x8, w8, torch.empty(4, 30, device=DEV, dtype=torch.bfloat16), swiglu=True)
    with pytest.raises(KernelError, match="head_dim"):
        K.attn_simple(rnd(1, 300 * 3), torch.empty(1, 300, device=DEV), torch.zeros(1, 2, 1, 64, 300, device=DEV),
                      torch.zeros(1, 1, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                      torch.zeros(1, dtype=torch.int32, device=DEV), 1, 1, 300, 64, None, 1.0)


@pytest.mark.parametrize("vocab", [331, 1000, 32768, 50001])
def test_argmax(K, vocab):
    lg = rnd(6, vocab, scale=3.0)
    lg[2, 7] = lg[2, vocab - 1] = 100.0                   # a tie: the lower index wins
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    K.argmax(lg, out)
    assert out.tolist() == [P.argmax_lowest(lg[i].cpu()) for i in range(6)] and out[2] == 7


@pytest.mark.parametrize("vocab", [331, 5000, 32768, 53600, 53700, 131072])      # rows of up to 53,6xx logits stay in shared memory
def test_sampling_chain(K, vocab):
    rows = 18
    lg = rnd(rows, vocab, scale=2.5, seed=4)
    g = torch.Generator().manual_seed(0)
    cases = []
    # the last three patterns keep the whole row in play when top-p comes: no top-k, or one of more candidates than a
    # block has threads (the cut of top-p is then found over the whole row, by passes over the probability mass)
    for i in range(rows):
        cases.append(dict(temperature=[0.8, 1.0, 0.0, 1.5, 0.3, 2.0, 0.8, 1.2, 0.6][i % 9],
                          top_k=[0, 50, 0, 5, 1, 200, 0, 2000, 0][i % 9],
                          top_p=[1.0, 0.9, 1.0, 0.5, 1.0, 0.95, 0.9, 0.8, 0.3][i % 9],
                          min_p=[0.0, 0.0, 0.0, 0.05, 0.0, 0.01, 0.0, 0.0, 0.001][i % 9],
                          repetition_penalty=[1.0, 1.3, 1.2, 1.0, 1.0, 1.1, 1.0, 1.1, 1.0][i % 9],
                          u=float(torch.rand((), generator=g))))
    hist = [[int(t) for t in torch.randint(0, vocab, (20,), generator=g)] + [3, 3, 3] for _ in range(rows)]
    bias = [[(5, 2.5), (9, -1.0), (5, 0.5)] if i % 3 == 0 else [] for i in range(rows)]
    from collections import Counter
    f = lambda key: torch.tensor([c[key] for c in cases], dtype=torch.float32, device=DEV)
    ho, ht, hc, bo, bt, bv = [0], [], [], [0], [], []
    for i in range(rows):
        for tok, cnt in Counter(hist[i]).items():
            ht.append(tok); hc.append(cnt)
        ho.append(len(ht))
        for tok, d in bias[i]:
            bt.append(tok); bv.append(d)
        bo.append(len(bt))
    ti = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    work = torch.empty_like(lg)
    K.sample(lg, work, out, f("temperature"), f("u"), top_k=ti([c["top_k"] for c in cases]), top_p=f("top_p"),
             min_p=f("min_p"), rep_penalty=f("repetition_penalty"), hist_off=ti(ho), hist_tok=ti(ht), hist_cnt=ti(hc),
             bias_off=ti(bo), bias_tok=ti(bt), bias_val=torch.tensor(bv, dtype=torch.float32, device=DEV))
    got = out.tolist()
    for i, c in enumerate(cases):
        kw = {k: v for k, v in c.items()}
        want = P.sample(lg[i].cpu(), history=hist[i], logit_bias=bias[i], **kw)
        if got[i] != want:
            # the draw may land within rounding of a boundary of the cumulative sum
            lo = P.sample(lg[i].cpu(), history=hist[i], logit_bias=bias[i], **dict(kw, u=max(0.0, c["u"] - 1e-5)))
            hi = P.sample(lg[i].cpu(), history=hist[i], logit_bias=bias[i], **dict(kw, u=min(1.0, c["u"] + 1e-5)))
            assert got[i] in (lo, hi), (i, c, got[i], want)


@pytest.mark.parametrize("n, width, k", [(8, 4096, 1024), (3, 331, 520), (64, 1000, 256), (1, 72, 64), (20, 16384, 128)])
@pytest.mark.parametrize("od", [torch.float32, torch.bfloat16])
def test_fused_reduce_residual_norm(K, n, width, k, od):
    """Partial products of a stream-k GEMM + residual + RMSNorm in one kernel, against the
    three kernels run one after the other."""
    x, w = rnd(n, k, dtype=torch.bfloat16, scale=0.5), rnd(width, k, dtype=torch.bfloat16, scale=0.2, seed=1)
    h0 = rnd(n, width, seed=2)
    nw = (1 + rnd(width, scale=0.1, seed=3)).bfloat16()
    h_ref = h0.clone()
    K.gemm_tc(x, w, h_ref, residual=h_ref, stream_k=True)
    out_ref = torch.empty(n, width, device=DEV, dtype=od)
    K.rmsnorm(h_ref, nw, out_ref, 1e-5)
    h = h0.clone()
    out = torch.full((n, width), 9.0, device=DEV, dtype=od)
    K.streamk_reduce_norm(K.gemm_tc_partial(x, w), h, nw, out, 1e-5)
    assert torch.equal(h, h_ref)
    tol = 2e-6 if od == torch.float32 else 1 / 128
    assert ((out.double() - out_ref.double()).abs() <= tol * out_ref.double().abs() + 1e-6).all()
    # gathered rows: h is left alone, rows may repeat or be absent
    idx = torch.tensor([n - 1, 0, -1, 0], dtype=torch.int32, device=DEV)
    h = h0.clone()
    out2 = torch.full((4, width), 9.0, device=DEV, dtype=od)
    K.streamk_reduce_norm(K.gemm_tc_partial(x, w), h, nw, out2, 1e-5, row_index=idx)
    assert torch.equal(h, h0)
    for r, srow in enumerate([n - 1, 0, -1, 0]):
        if srow < 0:
            assert float(out2[r].abs().max()) == 0.0
        else:
            assert ((out2[r].double() - out_ref[srow].double()).abs() <= tol * out_ref[srow].double().abs() + 1e-6).all()
    assert K.pending_partial is None


@pytest.mark.parametrize("pairing, hd, nqh, nkh", [("half", 128, 8, 2), ("adjacent", 48, 5, 3), ("half", 16, 4, 2)])
def test_fused_reduce_rope_cache_write(K, pairing, hd, nqh, nkh):
    """Partial products + rotation + cache write in one kernel, against product then rope_kv_write."""
    k, theta = 512, 1e4
    seqs = [(60, 10), (0, 3), (200, 1)]
    rows = sum(n for _, n in seqs) + 2
    pos = [p for b, n in seqs for p in range(b, b + n)] + [0, 0]
    seq = [i for i, (b, n) in enumerate(seqs) for _ in range(n)] + [-1, -1]
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    x = rnd(rows, k, dtype=torch.bfloat16, scale=0.5)
    w = rnd((nqh + 2 * nkh) * hd, k, dtype=torch.bfloat16, scale=0.2, seed=1)
    inv = P.inv_freq(hd, theta).to(DEV)
    cache_a, table = make_cache(3, [b + n for b, n in seqs], nkh, hd, torch.bfloat16)
    cache_b = cache_a.clone()
    qkv_a = torch.empty(rows, w.shape[0], device=DEV, dtype=torch.bfloat16)
    K.gemm_tc(x, w, qkv_a, stream_k=True)
    K.rope_kv_write(qkv_a, inv, t(pos), t(seq), table, cache_a, nqh, nkh, hd, hd, pairing == "adjacent", 64)
    qkv_b = torch.zeros(rows, w.shape[0], device=DEV, dtype=torch.bfloat16)
    K.streamk_reduce_rope_kv(K.gemm_tc_partial(x, w), qkv_b, inv, t(pos), t(seq), table, cache_b, nqh, nkh, hd, hd,
                             pairing == "adjacent", 64)
    K.check_device_errors()
    assert torch.equal(qkv_a[:-2], qkv_b[:-2]) and torch.equal(cache_a, cache_b)
    assert float(qkv_b[-2:].abs().max()) == 0.0              # padding rows are not written
    # the same with a row scale on the product's input: product + reduce with the scale, then the plain rotation
    from braidinfer_b200.csrc.api import RowScale
    sc = RowScale(shares_of(rnd(rows, 200, seed=5, scale=2.0), 3), 200, 1e-5)
    K.gemm_tc(x, w, qkv_a, stream_k=True, in_scale=sc)
    K.rope_kv_write(qkv_a, inv, t(pos), t(seq), table, cache_a, nqh, nkh, hd, hd, pairing == "adjacent", 64)
    K.streamk_reduce_rope_kv(K.gemm_tc_partial(x, w, in_scale=sc), qkv_b, inv, t(pos), t(seq), table, cache_b, nqh, nkh,
                             hd, hd, pairing == "adjacent", 64)
    K.check_device_errors()
    assert torch.equal(qkv_a[:-2], qkv_b[:-2]) and torch.equal(cache_a, cache_b)
