"""Each kernel alone against a plain float32 reference, at sizes other than the models'.

Where random inputs would hide a fault, the inputs are made so that it shows: one far key
among hundreds carries the whole softmax, keys sit exactly on a window's two edges, and every
sequence of a batch finds a value that names its own slot and position."""
import math

import numpy as np
import pytest
import torch

import plain_model as pm
import plain_sampling as ps
from sonicboom_b200 import ops
from sonicboom_b200.cache import Cache, KVNeed
from sonicboom_b200.engine.step import StepEntry, StepPlan
from sonicboom_b200.parts.feedforward import interleave_gate_up
from sonicboom_b200.sampling import Sampler, Sampling

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, ref, tol):
    err = pm.rel_err(got.float().cpu(), ref.float().cpu())
    assert err < tol, err


# --------------------------------------------------------------------------- small kernels

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    table = rnd(517, 72, dtype=DT[dtype])
    tokens = torch.tensor([0, 516, 3, 3, 100], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, device=DEV)
    ops.embed(tokens, table, out)
    assert torch.equal(out, table.float()[tokens.long()])
    # an id outside the table (what the sampler emits for logits that are not finite) reads
    # nothing and gives a row of NaN
    tokens = torch.tensor([-1, 2, 517, 2 ** 31 - 1], dtype=torch.int32, device=DEV)
    out = torch.zeros(4, 72, device=DEV)
    ops.embed(tokens, table, out)
    assert torch.isnan(out[[0, 2, 3]]).all() and torch.equal(out[1], table.float()[2])


@pytest.mark.parametrize("width", [8, 72, 1000, 3584])
@pytest.mark.parametrize("wdtype,odtype", [("float32", "float32"), ("bfloat16", "bfloat16"),
                                           ("float32", "bfloat16")])
def test_rmsnorm(width, wdtype, odtype):
    x = rnd(7, width, scale=3.0)
    w = rnd(width, dtype=DT[wdtype]) + 1
    out = torch.empty(7, width, dtype=DT[odtype], device=DEV)
    ops.rmsnorm(x, w, 1e-5, out)
    ref = pm.rms_norm(x.cpu(), w.float().cpu(), 1e-5)
    close(out, ref, 1e-6 if odtype == "float32" else 5e-3)
    rows = torch.tensor([6, 0, 6], dtype=torch.int32, device=DEV)
    g = torch.empty(3, width, dtype=DT[odtype], device=DEV)
    ops.rmsnorm(x, w, 1e-5, g, rows)
    assert torch.equal(g, out[rows.long()])
    # a row's result does not depend on the other rows of the launch
    one = torch.empty(1, width, dtype=DT[odtype], device=DEV)
    ops.rmsnorm(x[3:4].contiguous(), w, 1e-5, one)
    assert torch.equal(one[0], out[3])


def test_cast_round_trip():
    x = rnd(1000, 3)
    b = ops.cast(x, torch.bfloat16)
    assert torch.equal(b, x.to(torch.bfloat16)) and torch.equal(ops.cast(b, torch.float32), b.float())


# --------------------------------------------------------------------------------- products

def linear_ref(a, w, epilogue, bias, residual):
    y = a.double().cpu() @ w.double().cpu().t()
    if epilogue == ops.EPI_BIAS:
        y = y + bias.double().cpu()
    elif epilogue == ops.EPI_RESIDUAL:
        y = y + residual.double().cpu()
    elif epilogue == ops.EPI_SWIGLU:
        n = y.shape[1] // 2
        blocks = y.view(y.shape[0], n // 8, 2, 8)
        g, u = blocks[:, :, 0, :].reshape(-1, n), blocks[:, :, 1, :].reshape(-1, n)
        y = g / (1 + torch.exp(-g)) * u
    return y.float()


SHAPES = [(1, 24, 40), (3, 152, 72), (17, 1000, 200), (64, 96, 1024), (65, 264, 136),
          (200, 520, 328), (333, 128, 2048)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kernel", ["plain", "auto", "skinny", "tiled", "tc5"])
def test_linear_epilogues(M, N, K, dtype, kernel):
    if dtype == "float32" and kernel != "plain":
        pytest.skip("float32 has the plain kernel only")
    if kernel == "skinny" and M > 64:
        pytest.skip("the weight-streaming kernel takes at most 64 rows")
    dt = DT[dtype]
    a, w = rnd(M, K, dtype=dt), rnd(N, K, dtype=dt, scale=K ** -0.5, seed=1)
    bias, res = rnd(N, dtype=dt, seed=2), rnd(M, N, seed=3)
    tol = 1e-5      # float32 accumulation over up to 2048 terms (typical error sqrt(K) * 6e-8)
    for epi, odt in [(ops.EPI_NONE, torch.float32), (ops.EPI_BIAS, torch.float32),
                     (ops.EPI_RESIDUAL, torch.float32), (ops.EPI_SWIGLU, dt),
                     (ops.EPI_NONE, dt)]:
        if epi == ops.EPI_SWIGLU and N % 16:
            continue
        out = torch.empty(M, N // 2 if epi == ops.EPI_SWIGLU else N, dtype=odt, device=DEV)
        r = res.clone()
        ops.linear(a, w, out, epi, bias=bias if epi == ops.EPI_BIAS else None,
                   residual=r if epi == ops.EPI_RESIDUAL else None, kernel=kernel)
        close(out, linear_ref(a, w, epi, bias, res), tol if odt == torch.float32 else 5e-3)
        if epi == ops.EPI_RESIDUAL:                 # in place on the residual stream
            ops.linear(a, w, r, epi, residual=r, kernel=kernel)
            assert torch.equal(r, out)
    assert ops.tc5_status() == 0


@pytest.mark.parametrize("M", [1, 2, 7, 16, 33, 63, 64])
@pytest.mark.parametrize("scale", [1.0, 60.0])
def test_fused_gate_up_at_few_rows(M, scale):
    """SiLU(gate) * up from the decode form of the tcgen05 product, whose lanes share the tokens
    out in twos: odd and even numbers of rows, a last weight tile that is partly outside, and
    gates beyond -100 and 100 (the exponential overflows: the result is 0, or the up value times
    the gate)."""
    N, K = 1040, 200
    a = rnd(M, K, dtype=torch.bfloat16, scale=scale)
    w = rnd(N, K, dtype=torch.bfloat16, scale=K ** -0.5, seed=1)
    out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
    ops.linear(a, w, out, ops.EPI_SWIGLU, kernel="tc5")
    want = linear_ref(a, w, ops.EPI_SWIGLU, None, None)
    if scale > 1:
        gates = (a.double().cpu() @ w.double().cpu().T).view(M, N // 16, 2, 8)[:, :, 0]
        assert gates.min() < -100 and gates.max() > 100
    assert torch.isfinite(out).all()
    close(out, want, 5e-3)
    assert ops.tc5_status() == 0


def _every_epilogue(M, N, K):
    dt = torch.bfloat16
    a, w = rnd(M, K, dtype=dt), rnd(N, K, dtype=dt, scale=K ** -0.5, seed=1)
    bias, res = rnd(N, dtype=dt, seed=2), rnd(M, N, seed=3)
    outs = []
    for epi, odt in [(ops.EPI_NONE, torch.float32), (ops.EPI_BIAS, dt), (ops.EPI_RESIDUAL, torch.float32),
                     (ops.EPI_SWIGLU, dt)]:
        out = torch.empty(M, N // 2 if epi == ops.EPI_SWIGLU else N, dtype=odt, device=DEV)
        ops.linear(a, w, out, epi, bias=bias if epi == ops.EPI_BIAS else None,
                   residual=res.clone() if epi == ops.EPI_RESIDUAL else None, kernel="tc5")
        close(out, linear_ref(a, w, epi, bias, res), 1e-5 if odt == torch.float32 else 5e-3)
        outs.append(out)
    assert ops.tc5_status() == 0
    return outs


@pytest.mark.parametrize("M,N,K", [(1280, 3568, 72), (1280, 3344, 72), (1280, 3120, 72), (2048, 3568, 136),
                                   (200, 528, 328)])
def test_persistent_product_at_every_tile_width(M, N, K):
    """Sizes for which the persistent tcgen05 product with one block per tile picks each of its
    tile widths on 148 SMs (256, 240, 224, 208, 192), with a last tile that is only partly inside
    the matrix: every epilogue against the float64 product.  Widths that are odd multiples of 16
    end in a chunk of 16 columns."""
    ops.set_tc5_pairs(0)
    try:
        _every_epilogue(M, N, K)
    finally:
        ops.set_tc5_pairs(-1)


PAIR_SIZES = [(1280, 3376, 72, 256), (1280, 3152, 72, 240), (1280, 2928, 72, 224), (1280, 2720, 136, 208),
              (300, 560, 328, 192), (129, 528, 64, 192), (2048, 4608, 1032, 256), (2048, 3600, 136, 240)]


@pytest.mark.parametrize("M,N,K,width", PAIR_SIZES)
def test_product_on_pairs_of_sms(M, N, K, width):
    """The same product on clusters of two blocks (one MMA of 256 rows over two SMs), at sizes for
    which it picks each of its tile widths (the narrowest that gives the 74 pairs one wave when
    there are few rows; by the work per flop in the last two), all with a last tile that is partly
    outside the matrix: rows that end inside the first block's half of a tile (129), inside the second's (300:
    the second tile's second block loads nothing but zeros), several K tiles per stage of the
    ring (1,032 = 17 tiles, the last one of 8 values).  Every epilogue against the float64
    product, and the same bits as one block per tile gives."""
    ops.set_tc5_pairs(1)
    try:
        assert ops.tc5_tile_width(M, N) == width
        pairs = _every_epilogue(M, N, K)
        ops.set_tc5_pairs(0)
        single = _every_epilogue(M, N, K)
    finally:
        ops.set_tc5_pairs(-1)
    for a, b in zip(pairs, single):
        assert torch.equal(a, b)


@pytest.mark.parametrize("M,N,K", [(200, 528, 2048), (300, 400, 4096), (129, 3584, 1032), (512, 1040, 1200), (100, 1040, 2048)])
def test_product_with_few_rows_splits_k_over_the_pairs(M, N, K):
    """Few row tiles and a long inner dimension: the product on pairs of SMs shares every tile's K
    blocks out over the pairs that would have no tile (four, eight, two, two and four splits here),
    writes the partial sums to scratch and adds them in split order with the epilogue (also at 65 to
    128 rows, which otherwise run one block per tile).  Every
    epilogue against the float64 product; a last split that is shorter than the others, rows that
    end in the first block's half of a tile and a last tile that is partly outside the matrix."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ops.set_tc5_pairs(1)
    try:
        assert int(ops.lib().sb_gemm_tc5_scratch_bytes(M, N, K, sms)) > 0, "these sizes should split K"
        split = _every_epilogue(M, N, K)
        ops.set_tc5_pairs(0)
        whole = _every_epilogue(M, N, K)
    finally:
        ops.set_tc5_pairs(-1)
    for a, b in zip(split, whole):                     # another order of the same sum
        assert pm.rel_err(a.float().cpu(), b.float().cpu()) < (1e-5 if a.dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("kernel", ["plain", "skinny", "tiled", "tc5"])
def test_linear_rows_do_not_depend_on_the_batch(kernel):
    a, w = rnd(40, 256, dtype=torch.bfloat16), rnd(88, 256, dtype=torch.bfloat16, seed=1)
    full = torch.empty(40, 88, device=DEV)
    ops.linear(a, w, full, kernel=kernel)
    for rows in (slice(0, 1), slice(5, 12), slice(39, 40)):
        part = torch.empty(rows.stop - rows.start, 88, device=DEV)
        ops.linear(a[rows].contiguous(), w, part, kernel=kernel)
        assert pm.rel_err(part.cpu(), full[rows].cpu()) < 1e-6


def rmsnorm_ref(x, w, eps):
    x = x.double().cpu()
    return (x / torch.sqrt((x * x).mean(dim=1, keepdim=True) + eps) * w.double().cpu()).float()


@pytest.mark.parametrize("M,N,K", [(1, 1000, 512), (8, 3584, 1024), (13, 520, 2048), (33, 2052, 328),
                                   (64, 896, 4864), (8, 16388, 512), (8, 250, 512), (70, 512, 512)])
@pytest.mark.parametrize("ndtype", ["float32", "bfloat16"])
def test_linear_followed_by_a_norm(M, N, K, ndtype):
    """A product with the norm of its rows asked for: through the kernel that finishes the
    split-K product where it runs (up to 64 rows, widths that are multiples of 4 up to 16,384),
    else product then norm.  The product itself is the same to the bit either way."""
    a = rnd(M, K, dtype=torch.bfloat16)
    w = rnd(N, K, dtype=torch.bfloat16, scale=K ** -0.5, seed=1)
    bias, res = rnd(N, dtype=torch.bfloat16, seed=2), rnd(M, N, seed=3)
    nw = (1 + 0.3 * rnd(N, seed=4)).to(DT[ndtype])
    eps = 3e-5
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for epi in (ops.EPI_NONE, ops.EPI_BIAS, ops.EPI_RESIDUAL):
        kw = dict(bias=bias if epi == ops.EPI_BIAS else None)
        plain_out = torch.empty(M, N, device=DEV)
        ops.linear(a, w, plain_out, epi, residual=res.clone() if epi == ops.EPI_RESIDUAL else None,
                   kernel="tc5", **kw)
        out = res.clone() if epi == ops.EPI_RESIDUAL else torch.empty(M, N, device=DEV)
        normed = torch.empty(M, N, dtype=DT[ndtype], device=DEV)
        ops.linear(a, w, out, epi, residual=out if epi == ops.EPI_RESIDUAL else None,
                   norm=(nw, eps, normed), **kw)
        fuses = bool(ops.lib().sb_gemm_tc5_fuses_norm(M, N, K, sms, epi, 0, 0))
        assert fuses == (M <= 64 and N % 4 == 0 and N <= 16384 and K >= 512)   # K split at 8 tiles of 64
        if fuses:
            assert torch.equal(out, plain_out)
        close(out, linear_ref(a, w, epi, bias, res), 1e-5)
        close(normed, rmsnorm_ref(out, nw, eps), 1e-6 if ndtype == "float32" else 5e-3)   # bfloat16: half an ulp is 2^-8
    assert ops.tc5_status() == 0


def test_fused_gate_up_layout():
    gate, up = rnd(32, 8), rnd(32, 8, seed=1)
    f = interleave_gate_up(gate, up)
    assert torch.equal(f[0:8], gate[0:8]) and torch.equal(f[8:16], up[0:8])
    assert torch.equal(f[48:56], gate[24:32]) and torch.equal(f[56:64], up[24:32])


def test_linear_refuses_what_it_cannot_do():
    a, w = rnd(2, 8), rnd(24, 8)
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops.linear(a, w, torch.empty(2, 12, device=DEV), ops.EPI_SWIGLU)
    with pytest.raises(ops.KernelError, match="CUDA tensors only"):
        ops.linear(a.cpu(), w, torch.empty(2, 24, device=DEV))
    with pytest.raises(ops.KernelError, match="float32"):
        ops.linear(a, w, torch.empty(2, 24, dtype=torch.bfloat16, device=DEV), ops.EPI_RESIDUAL,
                   residual=torch.zeros(2, 24, device=DEV))


# ----------------------------------------------------------------- rotation + cache + attention

def make_cache(hkv, hd, window, dtype, max_tokens=2048):
    return Cache([KVNeed(hkv, hd, window)], [None], max_tokens, dtype, DEV)


def run_attention(cache, hq, hkv, hd, window, dtype, seqs, rot=None, theta=10000.0, scale=None,
                  kernel="auto"):
    """seqs: list of (slot, qkv float32 [n, (hq+2hkv)*hd]).  Writes k, v and returns attention
    output [rows, hq*hd] plus the rotated q."""
    rot = hd if rot is None else rot
    for s, x in seqs:
        cache.reserve(s, cache.length(s) + x.shape[0])
    plan = StepPlan(cache, [StepEntry(s, [0] * x.shape[0], []) for s, x in seqs], DEV)
    qkv = torch.cat([x for _, x in seqs]).to(DEV)
    i = np.arange(max(rot // 2, 1), dtype=np.float32)
    inv = torch.from_numpy(np.exp(-2.0 * i / np.float32(max(rot, 1)) * np.log(np.float32(theta)))
                           .astype(np.float32)).to(DEV)
    q = torch.empty(qkv.shape[0], hq, hd, dtype=dtype, device=DEV)
    g = plan.groups[0]
    storage = cache.groups[0].entry_storage(0)
    ops.rope_store(qkv, hq, hkv, hd, rot, inv, plan.row_seq, plan.row_pos, g.page_off, g.page_ids,
                   g.page_size, storage, q)
    out = torch.empty(qkv.shape[0], hq * hd, dtype=dtype, device=DEV)
    ops.attention(q, out, plan, 0, storage, hq, hkv, hd, window,
                  scale if scale is not None else hd ** -0.5, kernel=kernel)
    for s, x in seqs:
        cache.advance(s, cache.length(s) + x.shape[0])
    return out.float().cpu(), q.float().cpu()


def attention_ref(qkv, pos0, hq, hkv, hd, window, history=None, theta=10000.0, scale=None):
    """Plain implementation on one sequence; `history` is earlier rows' qkv."""
    allx = qkv if history is None else torch.cat([history, qkv])
    n = allx.shape[0]
    pos = torch.arange(n)
    q = pm.rope_neox(allx[:, :hq * hd].reshape(n, hq, hd), pos, theta)
    k = pm.rope_neox(allx[:, hq * hd:(hq + hkv) * hd].reshape(n, hkv, hd), pos, theta)
    v = allx[:, (hq + hkv) * hd:].reshape(n, hkv, hd)
    out = pm.attention(q, k, v, pos, pos, scale if scale is not None else hd ** -0.5, window)
    return out[n - qkv.shape[0]:].reshape(qkv.shape[0], hq * hd)


@pytest.mark.parametrize("hq,hkv,hd", [(4, 2, 16), (6, 1, 32), (5, 5, 48), (14, 2, 64), (28, 4, 128),
                                       (3, 1, 80), (8, 8, 256)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kernel", ["plain", "auto", "mma", "tma"])
def test_rotation_cache_and_attention(hq, hkv, hd, dtype, kernel):
    if dtype == "float32" and kernel != "plain":
        pytest.skip("float32 has the plain kernel only")
    if kernel == "tma" and hd not in (64, 128):
        pytest.skip("the persistent decode kernel is written for head sizes 64 and 128")
    if kernel == "mma" and hd not in (64, 128):
        pytest.skip("auto already is the mma.sync kernel at this head size")
    tol = 1e-5 if dtype == "float32" else 1.5e-2
    for window in (0, 37):
        cache = make_cache(hkv, hd, window, DT[dtype])
        lens = [1, 70, 150]
        xs = [torch.randn(n, (hq + 2 * hkv) * hd, generator=torch.Generator().manual_seed(n)) for n in lens]
        slots = [cache.open() for _ in lens]
        out, _ = run_attention(cache, hq, hkv, hd, window, DT[dtype], list(zip(slots, xs)), kernel=kernel)
        at = 0
        for x in xs:
            close(out[at:at + x.shape[0]], attention_ref(x, 0, hq, hkv, hd, window), tol)
            at += x.shape[0]
        # then decode: one more row for each sequence, then 3 more for one of them
        for n_new in (1, 3):
            news = [torch.randn(n_new, xs[0].shape[1], generator=torch.Generator().manual_seed(7 + i))
                    for i in range(len(xs))]
            out, _ = run_attention(cache, hq, hkv, hd, window, DT[dtype], list(zip(slots, news)),
                                   kernel=kernel)
            for i, (x, new) in enumerate(zip(xs, news)):
                close(out[i * n_new:(i + 1) * n_new],
                      attention_ref(new, x.shape[0], hq, hkv, hd, window, history=x), tol)
            xs = [torch.cat([x, new]) for x, new in zip(xs, news)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kernel", ["plain", "auto"])
def test_partial_rotation_and_no_rotation(dtype, kernel):
    if dtype == "float32" and kernel == "auto":
        pytest.skip("float32 has the plain kernel only")
    hq, hkv, hd = 4, 2, 32
    x = torch.randn(9, (hq + 2 * hkv) * hd, generator=torch.Generator().manual_seed(1))
    for rot in (0, 16):
        cache = make_cache(hkv, hd, 0, DT[dtype])
        _, q = run_attention(cache, hq, hkv, hd, 0, DT[dtype], [(cache.open(), x)], rot=rot, kernel=kernel)
        ref = x[:, :hq * hd].reshape(9, hq, hd).clone()
        if rot:
            ref[..., :rot] = pm.rope_neox(ref[..., :rot].contiguous(), torch.arange(9), 10000.0)
        close(q, ref, 1e-6 if dtype == "float32" else 5e-3)


def standout(n, hq, hkv, hd, key_pos, big=60.0):
    """qkv rows (no rotation is applied by the caller) where every query matches only the key
    at `key_pos`, strongly, and v rows spell (position + 1) in every component."""
    qkv = torch.zeros(n, (hq + 2 * hkv) * hd)
    qkv[:, :hq * hd] = 0.01 * torch.randn(n, hq * hd, generator=torch.Generator().manual_seed(5))
    qkv[:, 0:hq * hd:hd] = 1.0                            # component 0 of every query head
    k = qkv[:, hq * hd:(hq + hkv) * hd].view(n, hkv, hd)
    k[key_pos, :, 0] = big / (hd ** -0.5)
    v = qkv[:, (hq + hkv) * hd:].view(n, hkv, hd)
    v += (torch.arange(n, dtype=torch.float32) + 1)[:, None, None]
    return qkv


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kernel", ["plain", "auto"])
def test_a_far_key_among_hundreds_is_found(dtype, kernel):
    if dtype == "float32" and kernel == "auto":
        pytest.skip("float32 has the plain kernel only")
    hq, hkv, hd, n = 6, 2, 32, 700
    for key_pos in (3, 64, 255, 256, 511, 640):
        cache = make_cache(hkv, hd, 0, DT[dtype])
        s = cache.open()
        x = standout(n, hq, hkv, hd, key_pos)
        out, _ = run_attention(cache, hq, hkv, hd, 0, DT[dtype], [(s, x[:n - 1])], rot=0, kernel=kernel)
        last = out[-1]                                    # prefill row n-2 sees the key
        assert abs(float(last.mean()) - (key_pos + 1)) < 0.02 * (key_pos + 1), (key_pos, float(last.mean()))
        out, _ = run_attention(cache, hq, hkv, hd, 0, DT[dtype], [(s, x[n - 1:])], rot=0, kernel=kernel)
        assert abs(float(out.mean()) - (key_pos + 1)) < 0.02 * (key_pos + 1), (key_pos, float(out.mean()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kernel", ["plain", "auto"])
def test_window_edges(dtype, kernel):
    """Query i sees key j iff i - j < window: the key at i - window + 1 counts, i - window not."""
    if dtype == "float32" and kernel == "auto":
        pytest.skip("float32 has the plain kernel only")
    hq, hkv, hd, window = 4, 2, 16, 70
    for n in (71, 135, 200):                              # the last row is the query
        i = n - 1
        for key_pos, seen in ((i - window + 1, True), (i - window, False)):
            for decode in (False, True):
                cache = make_cache(hkv, hd, window, DT[dtype])
                s = cache.open()
                x = standout(n, hq, hkv, hd, key_pos)
                if decode:
                    run_attention(cache, hq, hkv, hd, window, DT[dtype], [(s, x[:i])], rot=0, kernel=kernel)
                    out, _ = run_attention(cache, hq, hkv, hd, window, DT[dtype], [(s, x[i:])], rot=0,
                                           kernel=kernel)
                else:
                    out, _ = run_attention(cache, hq, hkv, hd, window, DT[dtype], [(s, x)], rot=0,
                                           kernel=kernel)
                got = float(out[-1].mean())
                if seen:
                    assert abs(got - (key_pos + 1)) < 0.02 * (key_pos + 1), (n, key_pos, decode, got)
                else:                                     # an average over the window's own keys
                    assert i - window + 2 <= got <= i + 1, (n, key_pos, decode, got)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kernel", ["plain", "auto"])
def test_every_sequence_reads_its_own_pages(dtype, kernel):
    if dtype == "float32" and kernel == "auto":
        pytest.skip("float32 has the plain kernel only")
    hq, hkv, hd = 4, 1, 16
    cache = make_cache(hkv, hd, 0, DT[dtype], max_tokens=64 * 40)
    # interleave the sequences' growth so that their pages are interleaved in the pool
    slots = [cache.open() for _ in range(4)]
    lens = [130, 5, 260, 64]
    keys = [100, 2, 7, 63]
    xs = [standout(n + 1, hq, hkv, hd, k) for n, k in zip(lens, keys)]
    for i, x in enumerate(xs):                            # values name the sequence too
        x[:, (hq + hkv) * hd:] += 1000.0 * i
    fed = [0] * 4
    while any(f < n for f, n in zip(fed, lens)):
        step = [(s, x[f:min(f + 50, n)]) for s, x, f, n in zip(slots, xs, fed, lens) if f < n]
        run_attention(cache, hq, hkv, hd, 0, DT[dtype], step, rot=0, kernel=kernel)
        fed = [min(f + 50, n) for f, n in zip(fed, lens)]
    out, _ = run_attention(cache, hq, hkv, hd, 0, DT[dtype],
                           [(s, x[n:]) for s, x, n in zip(slots, xs, lens)], rot=0, kernel=kernel)
    for i, k in enumerate(keys):
        want = 1000.0 * i + k + 1
        assert abs(float(out[i].mean()) - want) < 0.01 * want + 0.5, (i, float(out[i].mean()), want)
    pages = [cache.page_list(s, 0) for s in slots]
    assert pages[0][1] != pages[0][0] + 1                 # the pool really was interleaved


@pytest.mark.parametrize("hq,hkv,hd,window,lens", [
    (28, 4, 128, 0, [700, 37]), (28, 4, 128, 100, [700, 333]), (8, 8, 128, 0, [513]),
    (7, 1, 64, 0, [1000]), (14, 2, 64, 37, [300, 5]), (6, 2, 64, 200, [450])])
def test_long_prefill_on_the_tensor_memory_kernel(hq, hkv, hd, window, lens):
    """Prompts of many pages, several query tiles per block, windows that start inside a page:
    the tcgen05 prefill kernel against the plain implementation; no wait in it may give up."""
    cache = make_cache(hkv, hd, window, torch.bfloat16, max_tokens=sum((n + 63) // 64 * 64 for n in lens))
    xs = [torch.randn(n, (hq + 2 * hkv) * hd, generator=torch.Generator().manual_seed(n)) for n in lens]
    slots = [cache.open() for _ in lens]
    out, _ = run_attention(cache, hq, hkv, hd, window, torch.bfloat16, list(zip(slots, xs)))
    at = 0
    for x in xs:
        close(out[at:at + x.shape[0]], attention_ref(x, 0, hq, hkv, hd, window), 1.5e-2)
        at += x.shape[0]
    assert ops.attention_status(hd) == 0


def test_prefill_continues_a_sequence_on_the_tensor_memory_kernel():
    """A second prompt chunk (positions do not start at 0) sees the first chunk's keys."""
    hq, hkv, hd = 14, 2, 128
    cache = make_cache(hkv, hd, 0, torch.bfloat16)
    s = cache.open()
    x = torch.randn(500, (hq + 2 * hkv) * hd, generator=torch.Generator().manual_seed(3))
    run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, [(s, x[:230])])
    out, _ = run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, [(s, x[230:])])
    close(out, attention_ref(x[230:], 230, hq, hkv, hd, 0, history=x[:230]), 1.5e-2)
    assert ops.attention_status(hd) == 0


@pytest.mark.parametrize("hq,hkv,hd,window", [(28, 4, 128, 0), (28, 4, 128, 300), (16, 8, 64, 0), (2, 1, 256, 0)])
def test_decode_steps_after_a_long_prompt(hq, hkv, hd, window):
    """Head sizes and groups of the benchmark model (and two others): a prompt of several
    splits, then single-token steps of two sequences of different lengths in one batch; every
    step against the plain implementation on the whole sequence."""
    cache = make_cache(hkv, hd, window, torch.bfloat16, max_tokens=2048)
    lens = [777, 130]
    xs = [torch.randn(n + 4, (hq + 2 * hkv) * hd, generator=torch.Generator().manual_seed(n)) for n in lens]
    slots = [cache.open() for _ in lens]
    run_attention(cache, hq, hkv, hd, window, torch.bfloat16, [(s, x[:n]) for s, x, n in zip(slots, xs, lens)])
    for step in range(4):
        out, _ = run_attention(cache, hq, hkv, hd, window, torch.bfloat16,
                               [(s, x[n + step:n + step + 1]) for s, x, n in zip(slots, xs, lens)])
        for i, (x, n) in enumerate(zip(xs, lens)):
            ref = attention_ref(x[n + step:n + step + 1], n + step, hq, hkv, hd, window, history=x[:n + step])
            close(out[i:i + 1], ref, 1.5e-2)
    assert ops.attention_status(hd) in (0, -1)            # -1: no tensor-memory kernel at this head size


@pytest.mark.parametrize("hq,hkv,hd,window", [(28, 4, 128, 0), (14, 2, 64, 0), (8, 8, 128, 100), (6, 2, 64, 37),
                                              (2, 1, 128, 0)])
def test_persistent_decode_kernel(hq, hkv, hd, window):
    """The persistent TMA decode kernel (forced: by itself it runs from about a wave of splits on):
    sequences of 5 to 4,200 keys in one step, so one split and many, 256-key and 512-key splits,
    a last tile with one key and with 64, three steps in a row; every row against the plain
    implementation, and bit for bit against the same step run alone (nothing but a sequence's own
    keys and length enters its result)."""
    lens = [700, 300, 1025, 64, 5, 257, 4200, 191]
    cache = make_cache(hkv, hd, window, torch.bfloat16, max_tokens=64 * 120)
    xs = [torch.randn(n + 3, (hq + 2 * hkv) * hd, generator=torch.Generator().manual_seed(n)) for n in lens]
    slots = [cache.open() for _ in lens]
    run_attention(cache, hq, hkv, hd, window, torch.bfloat16, [(s, x[:n]) for s, x, n in zip(slots, xs, lens)])
    alone = make_cache(hkv, hd, window, torch.bfloat16, max_tokens=64 * 70)
    s_alone = alone.open()
    run_attention(alone, hq, hkv, hd, window, torch.bfloat16, [(s_alone, xs[6][:lens[6]])])
    for step in range(3):
        out, _ = run_attention(cache, hq, hkv, hd, window, torch.bfloat16,
                               [(s, x[n + step:n + step + 1]) for s, x, n in zip(slots, xs, lens)], kernel="tma")
        for i, (x, n) in enumerate(zip(xs, lens)):
            ref = attention_ref(x[n + step:n + step + 1], n + step, hq, hkv, hd, window, history=x[:n + step])
            close(out[i:i + 1], ref, 1.5e-2)
        one, _ = run_attention(alone, hq, hkv, hd, window, torch.bfloat16,
                               [(s_alone, xs[6][lens[6] + step:lens[6] + step + 1])], kernel="tma")
        assert torch.equal(one[0], out[6])
    assert ops.attention_status(hd) == 0


def test_persistent_decode_kernel_finds_a_key_wherever_it_lies():
    """One key stands out; it lies in the first or the last tile of a split, in either half of a
    tile (the warps of a pair), in an even or an odd tile (the pairs), in the only tile."""
    hq, hkv, hd, n = 14, 2, 128, 901
    for key_pos in (3, 40, 64, 100, 255, 256, 300, 511, 640, 767, 899):
        cache = make_cache(hkv, hd, 0, torch.bfloat16)
        x = standout(n, hq, hkv, hd, key_pos)
        s = cache.open()
        run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, [(s, x[:n - 1])], rot=0)
        out, _ = run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, [(s, x[n - 1:])], rot=0, kernel="tma")
        assert abs(float(out.mean()) - (key_pos + 1)) < 0.02 * (key_pos + 1), (key_pos, float(out.mean()))


@pytest.mark.parametrize("kernel", ["tma", "mma"])
def test_decode_over_forty_splits(kernel):
    """A sequence of 20,001 keys (40 splits of 512) beside one of 9,000 (18) and a short one: the
    merge of the splits goes through several rounds of loads and, after the persistent kernel,
    through thread groups with ten, ten, ten and ten splits (five, five, five and three for the
    second sequence).  One key stands out, in the first, a middle or the last split; then
    random rows against the plain implementation."""
    hq, hkv, hd = 4, 2, 128
    lens = [20001, 9000, 70]
    for key_pos in (5, 5000, 10300, 15500, 19990):
        cache = make_cache(hkv, hd, 0, torch.bfloat16, max_tokens=64 * 320)
        x = standout(lens[0], hq, hkv, hd, key_pos)
        s = cache.open()
        run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, [(s, x[:-1])], rot=0)
        out, _ = run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, [(s, x[-1:])], rot=0, kernel=kernel)
        assert abs(float(out.mean()) - (key_pos + 1)) < 0.02 * (key_pos + 1), (key_pos, float(out.mean()))
    cache = make_cache(hkv, hd, 0, torch.bfloat16, max_tokens=64 * 470)
    xs = [torch.randn(n + 1, (hq + 2 * hkv) * hd, generator=torch.Generator().manual_seed(n)) * 0.5 for n in lens]
    slots = [cache.open() for _ in lens]
    for s, x, n in zip(slots, xs, lens):
        run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, [(s, x[:n])])
    out, _ = run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, [(s, x[n:]) for s, x, n in zip(slots, xs, lens)],
                           kernel=kernel)
    for i, (x, n) in enumerate(zip(xs, lens)):
        close(out[i:i + 1], attention_ref(x[n:], n, hq, hkv, hd, 0, history=x[:n]), 1.5e-2)
    assert ops.attention_status(hd) == 0


def test_many_sequences_reach_the_persistent_decode_kernel_by_themselves():
    """96 sequences x 4 key/value heads x 8 splits (one sequence of 1,900 keys sizes the grid, the
    others have 100 to 700): more than ten splits per SM on 148 SMs, so "auto" is the
    persistent kernel, which finds most of its work items empty; its rows equal the forced
    kernel's bit for bit, differ from the earlier kernel's by rounding only, and match the plain
    implementation."""
    hq, hkv, hd = 8, 4, 128
    g = torch.Generator().manual_seed(5)
    lens = [1900] + torch.randint(100, 700, (95,), generator=g).tolist()
    cache = make_cache(hkv, hd, 0, torch.bfloat16, max_tokens=(31 + 95 * 12) * 64)
    xs = [torch.randn(n + 1, (hq + 2 * hkv) * hd, generator=torch.Generator().manual_seed(n)) * 0.5 for n in lens]
    slots = [cache.open() for _ in lens]
    run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, [(s, x[:n]) for s, x, n in zip(slots, xs, lens)])
    step = [(s, x[n:]) for s, x, n in zip(slots, xs, lens)]
    outs = {}
    for kernel in ("auto", "tma", "mma"):
        outs[kernel], _ = run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, step, kernel=kernel)
        for s, n in zip(slots, lens):                 # the step is run three times: take it back
            cache.truncate(s, n)
    assert torch.equal(outs["auto"], outs["tma"])
    assert not torch.equal(outs["auto"], outs["mma"]) and pm.rel_err(outs["auto"], outs["mma"]) < 1e-2
    for i in (0, 17, 95):
        ref = attention_ref(xs[i][lens[i]:], lens[i], hq, hkv, hd, 0, history=xs[i][:lens[i]])
        close(outs["auto"][i:i + 1], ref, 1.5e-2)


def test_decode_attention_across_the_split_length_change():
    """Splits are 256 keys up to a sequence length of 4,096 and 512 beyond.  A sequence that
    grows from 4,094 to 4,099 keys crosses the change, next to a short one in the same batch;
    every step against the plain implementation, and the far key at position 3 is still found."""
    hq, hkv, hd = 4, 1, 64
    cache = make_cache(hkv, hd, 0, torch.bfloat16, max_tokens=4096 + 256 + 128)
    lens = [4093, 200]
    xs = [torch.randn(n + 6, (hq + 2 * hkv) * hd, generator=torch.Generator().manual_seed(n)) for n in lens]
    slots = [cache.open() for _ in lens]
    run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, [(s, x[:n]) for s, x, n in zip(slots, xs, lens)])
    for step in range(6):
        out, _ = run_attention(cache, hq, hkv, hd, 0, torch.bfloat16,
                               [(s, x[n + step:n + step + 1]) for s, x, n in zip(slots, xs, lens)])
        for i, (x, n) in enumerate(zip(xs, lens)):
            ref = attention_ref(x[n + step:n + step + 1], n + step, hq, hkv, hd, 0, history=x[:n + step])
            close(out[i:i + 1], ref, 1.5e-2)
    cache2 = make_cache(hkv, hd, 0, torch.bfloat16, max_tokens=4096 + 256)
    x = standout(4200, hq, hkv, hd, 3)
    s = cache2.open()
    run_attention(cache2, hq, hkv, hd, 0, torch.bfloat16, [(s, x[:4199])], rot=0)
    out, _ = run_attention(cache2, hq, hkv, hd, 0, torch.bfloat16, [(s, x[4199:])], rot=0)
    assert abs(float(out.mean()) - 4.0) < 0.08, float(out.mean())


def test_a_far_key_is_found_by_the_tensor_memory_kernel():
    hq, hkv, hd, n = 8, 2, 64, 900
    for key_pos in (3, 64, 255, 511, 640, 895):
        cache = make_cache(hkv, hd, 0, torch.bfloat16)
        x = standout(n, hq, hkv, hd, key_pos)
        out, _ = run_attention(cache, hq, hkv, hd, 0, torch.bfloat16, [(cache.open(), x)], rot=0)
        last = out[-1]
        assert abs(float(last.mean()) - (key_pos + 1)) < 0.02 * (key_pos + 1), (key_pos, float(last.mean()))
        first = out[key_pos]                              # the row of the key itself sees it too
        assert abs(float(first.mean()) - (key_pos + 1)) < 0.02 * (key_pos + 1)


# --------------------------------------------------------------------------------- sampling

def test_sampler_matches_the_plain_sampler():
    sampler = Sampler(DEV)
    g = torch.Generator().manual_seed(0)
    for vocab in (50, 256, 1003, 152064):
        logits = (torch.randn(6, vocab, generator=g) * 3).to(DEV)
        logits[1, :] = 0.25                               # all tied: lowest ids win
        logits[2, vocab // 2] = 40.0
        hist = [list(range(0, 40)), [1, 1, 2], [vocab // 2] * 5, [], [3, 4], [vocab - 1]]
        cases = [Sampling(), Sampling(temperature=0.8, seed=5), Sampling(temperature=1.5, top_k=7, seed=1),
                 Sampling(temperature=1.0, top_p=0.7, seed=2 ** 50), Sampling(temperature=0.6, min_p=0.1, seed=3),
                 Sampling(temperature=0.9, seed=4, repeat_penalty=1.3, presence_penalty=0.5,
                          frequency_penalty=0.25, repeat_last_n=16),
                 Sampling(repeat_penalty=5.0, presence_penalty=100.0)]
        for s in cases:
            s = s.checked()
            before = logits.clone()
            for position in (0, 17, 2 ** 33 + 1):
                got = sampler.sample(logits, [s] * 6, [position + r for r in range(6)], hist)
                want = [ps.sample_token(logits[r].cpu().numpy(),
                                        ps.Params(s.temperature, s.top_k, s.top_p, s.min_p, s.seed,
                                                  s.repeat_penalty, s.repeat_last_n, s.presence_penalty,
                                                  s.frequency_penalty), position + r, hist[r])
                        for r in range(6)]
                assert got == want, (vocab, s, position)
            assert torch.equal(logits, before)            # penalties were undone


def test_logits_that_are_not_finite_are_an_error_not_a_token():
    sampler = Sampler(DEV)
    logits = torch.randn(3, 300).to(DEV)
    logits[1, :] = float("nan")
    with pytest.raises(ops.KernelError, match="row 1"):
        sampler.sample(logits, [Sampling(temperature=0.7, seed=1).checked()] * 3, [0, 1, 2], [[], [], []])
    logits[1, :] = 0.0
    assert all(0 <= t < 300 for t in sampler.sample(
        logits, [Sampling(temperature=0.7, seed=1).checked()] * 3, [0, 1, 2], [[], [], []]))


def test_sampled_tokens_do_not_depend_on_the_row():
    sampler = Sampler(DEV)
    logits = (torch.randn(4, 500, generator=torch.Generator().manual_seed(2)) * 2).to(DEV)
    s = Sampling(temperature=1.0, seed=9).checked()
    a = sampler.sample(logits, [s] * 4, [10, 11, 12, 13], [[]] * 4)
    b = sampler.sample(logits.flip(0).contiguous(), [s] * 4, [13, 12, 11, 10], [[]] * 4)
    assert a == b[::-1]


@pytest.mark.parametrize("hq,hkv,hd,K,rot", [(28, 4, 128, 3584, 128), (6, 2, 64, 192, 64), (8, 2, 64, 2048, 32),
                                             (4, 4, 128, 1024, 0)])
@pytest.mark.parametrize("rows", [3, 9, 33, 64, 70])
def test_fused_projection_rotation_and_cache_write(hq, hkv, hd, K, rot, rows):
    """`qkv_rope_store` (where the split-K product's reduce kernel also rotates and writes the
    cache: 9 to 64 rows of the larger sizes) against the product and `rope_store` one after the
    other: the same queries and the same cache pages, for rows of several sequences at unequal
    positions, with a partly rotated head, without rotation, and for queries only."""
    dt = torch.bfloat16
    N = (hq + 2 * hkv) * hd
    a, w = rnd(rows, K, dtype=dt), rnd(N, K, dtype=dt, scale=K ** -0.5, seed=1)
    bias = rnd(N, dtype=dt, seed=2)
    inv = torch.from_numpy(np.exp(-2.0 * np.arange(max(rot // 2, 1), dtype=np.float32) / np.float32(max(rot, 1))
                                  * np.log(np.float32(10000.0))).astype(np.float32)).to(DEV)
    lens = [rows - 2 * (rows // 3), rows // 3, rows // 3] if rows >= 3 else [rows]
    results = []
    for fused in (True, False):
        cache = make_cache(hkv, hd, 0, dt, max_tokens=64 * 8)
        slots = [cache.open() for _ in lens]
        for i, (s, n) in enumerate(zip(slots, lens)):      # unequal starting positions
            cache.reserve(s, 37 * i + n)
            cache.advance(s, 37 * i)
        plan = StepPlan(cache, [StepEntry(s, [0] * n, []) for s, n in zip(slots, lens)], DEV)
        g = plan.groups[0]
        storage = cache.groups[0].entry_storage(0)
        q = torch.empty(rows, hq, hd, dtype=dt, device=DEV)
        if fused:
            ops.qkv_rope_store(a, w, bias, hq, hkv, hd, rot, inv, plan.row_seq, plan.row_pos, g.page_off,
                               g.page_ids, g.page_size, storage, q)
        else:
            qkv = torch.empty(rows, N, device=DEV)
            ops.linear(a, w, qkv, ops.EPI_BIAS, bias=bias)
            ops.rope_store(qkv, hq, hkv, hd, rot, inv, plan.row_seq, plan.row_pos, g.page_off, g.page_ids,
                           g.page_size, storage, q)
        results.append((q.float().cpu(), storage.float().cpu()))
    (q1, c1), (q2, c2) = results
    assert float(c2.abs().max()) > 0
    # the same product (to the last bit when the same kernel computes it; the split-K form adds
    # its partial tiles in another order) and the same rotation arithmetic in every kernel
    assert pm.rel_err(q1, q2) < 4e-3 and pm.rel_err(c1, c2) < 4e-3       # an ulp of bfloat16 at most
    # queries only (a layer that reads another layer's cache)
    qa, qb = torch.empty(rows, hq, hd, dtype=dt, device=DEV), torch.empty(rows, hq, hd, dtype=dt, device=DEV)
    plan = StepPlan(cache, [StepEntry(s, [0] * n, []) for s, n in zip(slots, lens)], DEV)
    ops.qkv_rope_store(a, w[:hq * hd], bias[:hq * hd], hq, hkv, hd, rot, inv, plan.row_seq, plan.row_pos, None,
                       None, 64, None, qa)
    qkv = torch.empty(rows, hq * hd, device=DEV)
    ops.linear(a, w[:hq * hd].contiguous(), qkv, ops.EPI_BIAS, bias=bias[:hq * hd].contiguous())
    ops.rope_store(qkv, hq, hkv, hd, rot, inv, plan.row_seq, plan.row_pos, None, None, 64, None, qb)
    assert pm.rel_err(qa.float().cpu(), qb.float().cpu()) < 4e-3
    assert ops.tc5_status() == 0


# ------------------------------------------------ positions outside a sequence's own pages
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hq,hkv,hd,rows", [(4, 2, 16, 3), (28, 4, 128, 3), (4, 2, 16, 80), (8, 4, 64, 60)])
def test_a_position_without_a_page_of_its_own_writes_and_reads_nothing(dtype, hq, hkv, hd, rows):
    """Rows whose position lies beyond their sequence's page list (a plan that a finished row of
    a captured batch would reach if nothing stopped it), or before 0: the rotation kernel writes
    no key or value for them, the attention gives them rows of zeros, every other sequence's
    pages stay as they were, and the neighbours' results are what they are without them.  All
    three forms of the rotation kernel (per head, per row, vector), the decode attention's merge
    counters and (60 sequences x 4 heads x 2 splits) the persistent decode kernel are covered: a
    second, ordinary step right after gives the right result."""
    dt = DT[dtype]
    cache = make_cache(hkv, hd, 0, dt, max_tokens=64 * 7 * rows)
    storage = cache.groups[0].entry_storage(0)
    slots = [cache.open() for _ in range(rows)]
    width = (hq + 2 * hkv) * hd
    base = 300                                              # two key splits in the decode kernel
    hist = [rnd(base + i, width, seed=30 + i).cpu() for i in range(rows)]
    run_attention(cache, hq, hkv, hd, 0, dt, [(s, h) for s, h in zip(slots, hist)])
    new = [rnd(1, width, seed=60 + i).cpu() for i in range(rows)]
    for s in slots:
        cache.reserve(s, cache.length(s) + 1)
    plan = StepPlan(cache, [StepEntry(s, [0], []) for s in slots], DEV)
    n_pg = [len(cache.page_list(s, 0)) for s in slots]
    # the first and the last row: just beyond their own pages and far beyond; the second: before 0
    bad = {0: 64 * n_pg[0], rows - 1: 64 * 2 * n_pg[-1] + 3, 1: -1}
    pos = plan.row_pos.clone()
    for r, p in bad.items():
        pos[r] = p
    plan.row_pos.copy_(pos)                                 # seq_pos0 is the same memory only in a decode plan
    plan.seq_pos0.copy_(pos)
    before = storage.clone()
    qkv = torch.cat(new).to(DEV)
    inv = torch.from_numpy(np.exp(-2.0 * np.arange(hd // 2, dtype=np.float32) / np.float32(hd)
                                  * np.log(np.float32(10000.0))).astype(np.float32)).to(DEV)
    q = torch.empty(rows, hq, hd, dtype=dt, device=DEV)
    g = plan.groups[0]
    ops.rope_store(qkv, hq, hkv, hd, hd, inv, plan.row_seq, plan.row_pos, g.page_off, g.page_ids,
                   g.page_size, storage, q)
    changed = (storage != before).any(dim=-1).any(dim=-1)             # [page, k|v, head]
    good_pages = {cache.page_list(s, 0)[(base + i) // 64] for i, s in enumerate(slots) if i not in bad}
    assert set(changed.nonzero()[:, 0].tolist()) == good_pages
    kernels = ["auto", "tma"] if dtype == "bfloat16" and hd in (64, 128) else ["auto"]
    for kernel in kernels:                                  # both decode kernels where there are two
        out = torch.full((rows, hq * hd), 7.0, dtype=dt, device=DEV)
        ops.attention(q, out, plan, 0, storage, hq, hkv, hd, 0, hd ** -0.5, kernel=kernel)
        torch.cuda.synchronize()
        out = out.float().cpu()
        for r in range(rows):
            if r in bad:
                assert float(out[r].abs().max()) == 0.0, (kernel, r)
            else:
                ref = attention_ref(new[r], base + r, hq, hkv, hd, 0, history=hist[r])
                close(out[r:r + 1], ref, 1e-5 if dtype == "float32" else 2e-2)
    # the same step with its true positions right after: scratch and counters are as they should be
    plan2 = StepPlan(cache, [StepEntry(s, [0], []) for s in slots], DEV)
    g2 = plan2.groups[0]
    ops.rope_store(qkv, hq, hkv, hd, hd, inv, plan2.row_seq, plan2.row_pos, g2.page_off, g2.page_ids,
                   g2.page_size, storage, q)
    out2 = torch.empty(rows, hq * hd, dtype=dt, device=DEV)
    ops.attention(q, out2, plan2, 0, storage, hq, hkv, hd, 0, hd ** -0.5)
    for r in range(rows):
        ref = attention_ref(new[r], base + r, hq, hkv, hd, 0, history=hist[r])
        close(out2[r:r + 1].float().cpu(), ref, 1e-5 if dtype == "float32" else 2e-2)


# ------------------------------------------------------------------ seeded random tensors
@pytest.mark.parametrize("n", [1, 3, 4, 5, 257, 1_000_003])
def test_random_tensors_are_the_same_bits_on_the_device_and_in_numpy(n):
    """The kernel restates weights/random_init.normal_numpy step for step with individually
    rounded float32 operations: float32 output is equal bit for bit, bfloat16 output equals the
    rounded numpy values, for other means and deviations too."""
    from sonicboom_b200.weights import random_init as ri
    for seed, name, mean, std in [(0, "a", 0.0, 1.0), (2 ** 40 + 5, "model.norm.weight", 1.0, 0.05),
                                  (11, "lm_head.weight", 0.0, 0.02)]:
        key = ri.tensor_key(seed, name)
        want = torch.from_numpy(ri.normal_numpy(n, *key, mean, std))
        got = ops.random_normal(torch.empty(n, dtype=torch.float32, device=DEV), *key, mean, std).cpu()
        differs = got.view(torch.int32) != want.view(torch.int32)
        assert not bool((differs & (want != 0)).any()), int(differs.sum())   # a zero may differ in its sign
        assert torch.equal(got, want)
        got16 = ops.random_normal(torch.empty(n, dtype=torch.bfloat16, device=DEV), *key, mean, std).cpu()
        assert torch.equal(got16, want.to(torch.bfloat16))


def test_a_model_made_on_the_device_equals_the_folder_written_without_one(tmp_path):
    import sonicboom_b200 as sb
    from conftest import INIT, TINY
    from sonicboom_b200.models import tensor_requests
    from sonicboom_b200.config import spec_from_config_dict
    from sonicboom_b200.weights import RandomSource, SafetensorsDir
    sb.write_random_model(tmp_path, TINY["C"], seed=17, **INIT["C"])
    folder = SafetensorsDir(tmp_path)
    _, spec = spec_from_config_dict(TINY["C"])
    src = RandomSource(tensor_requests(spec), 17, device=DEV, **INIT["C"])
    assert sorted(src.names()) == sorted(folder.names())
    for name in src.names():
        assert torch.equal(src.tensor(name).cpu(), folder.tensor(name)), name
    # and the model: the same logits from the folder and from the seed
    a = sb.Engine(sb.load_model(tmp_path, dtype="float32"), max_tokens=128)
    b = sb.Engine(sb.random_model(TINY["C"], 17, dtype="float32", **INIT["C"]), max_tokens=128)
    toks = list(range(3, 60))
    la = a.step([(a.open(), toks, [len(toks) - 1])])
    lb = b.step([(b.open(), toks, [len(toks) - 1])])
    assert torch.equal(la, lb)
