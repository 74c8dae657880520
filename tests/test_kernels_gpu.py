"""Each kernel alone against a plain float64 reference, at sizes other than the
engine tests': widths and vocabularies that are no power of two, head sizes in
steps of 16, odd numbers of heads and groups, scattered cache blocks."""

import numpy as np
import pytest
import torch

import plain_model as plain
from semantic_aware_adaptive_kv_cache_precision_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
ULP = {torch.float32: 2.0 ** -23, torch.bfloat16: 2.0 ** -8}


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a)).to(DEV).to(dtype).contiguous()


def host(t):
    return t.detach().double().cpu().numpy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    rng = np.random.default_rng(0)
    table = dev(rng.standard_normal((301, 70)), dtype)
    ids = torch.tensor([0, 300, 5, 301, -1, 17], dtype=torch.int32, device=DEV)
    out = ops.embed(ids, table)
    assert out.dtype == torch.float32
    want = host(table)[[0, 300, 5, 0, 0, 17]]
    want[3] = want[4] = 0.0                     # ids outside the table give zero rows
    np.testing.assert_array_equal(host(out), want)


@pytest.mark.parametrize("hidden", [48, 200, 1536, 5001])
@pytest.mark.parametrize("wdtype,odtype", [(torch.float32, torch.float32),
                                           (torch.bfloat16, torch.bfloat16),
                                           (torch.float32, torch.bfloat16)])
def test_rms_norm(hidden, wdtype, odtype):
    rng = np.random.default_rng(hidden)
    x = dev(rng.standard_normal((7, hidden)) * 3.0)
    w = dev(1 + 0.1 * rng.standard_normal(hidden), wdtype)
    eps = 1e-5
    want = plain.rms_norm(host(x), host(w), eps)
    got = ops.rms_norm(x, w, eps, odtype)
    np.testing.assert_allclose(host(got), want, rtol=2 * ULP[odtype], atol=1e-30)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    picked = ops.rms_norm(x, w, eps, odtype, rows=rows)
    assert torch.equal(picked, got[[6, 0, 3]])          # rows are independent, to the bit
    # eps matters when the row is tiny
    tiny = dev(np.full((1, hidden), 1e-4))
    np.testing.assert_allclose(host(ops.rms_norm(tiny, w, 1e-2, torch.float32)),
                               plain.rms_norm(host(tiny), host(w), 1e-2), rtol=1e-5)


@pytest.mark.parametrize("hidden", [128, 1536, 2048, 3584, 4096, 200])
@pytest.mark.parametrize("parts", [0, 1, 3])
def test_rms_norm_of_many_rows(hidden, parts):
    """From 256 rows on, bf16 norms run a warp a row (hidden a multiple of 128, up to 4,096;
    other sizes keep the block-a-row kernel): against float64, with a sum of `parts` products
    folded into the stream on the way, with a gather of rows, and equal to the bit to what
    the few-rows kernel gives each row by itself."""
    rng = np.random.default_rng(hidden + parts)
    n = 300
    x = dev(rng.standard_normal((n, hidden)) * 2.0)
    w = dev(1 + 0.1 * rng.standard_normal(hidden), torch.bfloat16)
    eps = 1e-6
    if parts:
        add = dev(rng.standard_normal((parts, n, hidden)))
        total = host(x) + host(add).sum(0)
        stream = x.clone()
        got = ops.rms_norm(stream, w, eps, torch.bfloat16, add=add if parts > 1 else add[0])
        np.testing.assert_allclose(host(stream), total, rtol=1e-6, atol=1e-6)    # x keeps the sum
        few = x[:5].clone()
        part = add[:, :5].contiguous()
        ops.rms_norm(few, w, eps, torch.bfloat16, add=part if parts > 1 else part[0])
        assert torch.equal(few, stream[:5])         # the same sum, in the same order
    else:
        total = host(x)
        got = ops.rms_norm(x, w, eps, torch.bfloat16)
        rows = torch.as_tensor(rng.permutation(n)[:280].astype(np.int32)).to(DEV)
        picked = ops.rms_norm(x, w, eps, torch.bfloat16, rows=rows)
        assert torch.equal(picked, got[rows.long()])
    # (the fp32 sums of up to four terms of size <= 10 are off by up to 4 * 2^-24 * 10, which
    # an element that cancels to nearly nothing shows as a large RELATIVE error: hence the atol)
    np.testing.assert_allclose(host(got), plain.rms_norm(total, host(w), eps),
                               rtol=2 * ULP[torch.bfloat16], atol=3e-6)


def make_cache(rng, n_blocks, kv_heads, head_dim, dtype):
    k = dev(rng.standard_normal((n_blocks, kv_heads, ops.CACHE_BLOCK, head_dim)), dtype)
    v = dev(rng.standard_normal((n_blocks, kv_heads, ops.CACHE_BLOCK, head_dim)), dtype)
    return k, v


def gather_cache(cache, table_row, length):
    """[length, kv_heads, head_dim] float64 of one sequence from its blocks."""
    c = host(cache)
    rows = [c[table_row[p // 64], :, p % 64, :] for p in range(length)]
    return np.stack(rows)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,rot", [(4, 2, 16, 16), (6, 3, 48, 32),
                                                         (5, 1, 128, 128), (2, 2, 256, 64)])
def test_rope_store(dtype, heads, kv_heads, head_dim, rot):
    rng = np.random.default_rng(heads * head_dim)
    starts, counts = [0, 130, 63], [70, 1, 3]           # three sequences, one in mid-decode
    T = sum(counts)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = dev(rng.standard_normal((T, width)), dtype)
    before = host(qkv)
    positions = np.concatenate([np.arange(s, s + c) for s, c in zip(starts, counts)])
    token_seq = np.repeat(np.arange(3), counts)
    table = np.array([[5, 2, -1, -1], [7, 0, 3, -1], [1, 6, -1, -1]], dtype=np.int32)
    k_cache, v_cache = make_cache(rng, 8, kv_heads, head_dim, dtype)
    k0, v0 = host(k_cache).copy(), host(v_cache).copy()
    theta = 1e4
    j = np.arange(rot // 2)
    angle = np.arange(256)[:, None] * np.power(theta, -2.0 * j / rot)[None, :]
    cos, sin = dev(np.cos(angle)), dev(np.sin(angle))
    ops.rope_store(qkv, dev(positions, torch.int32), dev(token_seq, torch.int32),
                   dev(table, torch.int32), cos, sin, k_cache, v_cache, heads, kv_heads, head_dim)
    c, s = host(cos)[positions], host(sin)[positions]

    def rotate(x):                                        # x [T, h, d]
        out = x.copy()
        out[..., :rot] = plain.rotate_half(x[..., :rot], c, s)
        return out

    q_want = rotate(before[:, :heads * head_dim].reshape(T, heads, head_dim))
    k_want = rotate(before[:, heads * head_dim:(heads + kv_heads) * head_dim]
                    .reshape(T, kv_heads, head_dim))
    v_want = before[:, (heads + kv_heads) * head_dim:].reshape(T, kv_heads, head_dim)
    tol = dict(rtol=0, atol=4 * ULP[dtype] * 4)
    np.testing.assert_allclose(host(qkv)[:, :heads * head_dim].reshape(T, heads, head_dim),
                               q_want, **tol)
    np.testing.assert_array_equal(host(qkv)[:, heads * head_dim:], before[:, heads * head_dim:])
    k1, v1 = host(k_cache), host(v_cache)
    touched = np.zeros(k1.shape[:1] + k1.shape[2:3], dtype=bool)      # [block, offset]
    for t in range(T):
        b, o = table[token_seq[t], positions[t] // 64], positions[t] % 64
        np.testing.assert_allclose(k1[b, :, o, :], k_want[t], **tol)
        np.testing.assert_array_equal(v1[b, :, o, :], v_want[t])
        touched[b, o] = True
    # nothing else in the cache changed
    untouched = ~touched
    for now, was in ((k1, k0), (v1, v0)):
        np.testing.assert_array_equal(now.transpose(0, 2, 1, 3)[untouched],
                                      was.transpose(0, 2, 1, 3)[untouched])


def attention_reference(q, k, v, pos, heads, kv_heads, scale, window):
    """One query [heads, d] at position pos over keys [len, kv_heads, d]."""
    out = np.empty_like(q)
    first = max(0, pos - window + 1) if window else 0
    for h in range(heads):
        g = h // (heads // kv_heads)
        s = (k[first:pos + 1, g] @ q[h]) * scale
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ v[first:pos + 1, g]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [
    (4, 2, 16, None), (6, 1, 32, None), (7, 7, 80, None), (12, 2, 128, 100), (3, 3, 256, 64),
    (10, 5, 112, 1)])
def test_attention_plain(dtype, heads, kv_heads, head_dim, window):
    rng = np.random.default_rng(head_dim + heads)
    # sequences: a 150-token prefill, a decode at position 299, a 2-token chunk after 64
    starts, counts = [0, 299, 64], [150, 1, 2]
    table = np.array([[9, 4, 11, -1, -1], [0, 8, 2, 6, 10], [3, 7, -1, -1, -1]], dtype=np.int32)
    k_cache, v_cache = make_cache(rng, 12, kv_heads, head_dim, dtype)
    T = sum(counts)
    q = dev(rng.standard_normal((T, heads * head_dim)), dtype)
    positions = np.concatenate([np.arange(s, s + c) for s, c in zip(starts, counts)])
    token_seq = np.repeat(np.arange(3), counts)
    scale = head_dim ** -0.5
    got = ops.attention_plain(q, k_cache, v_cache, dev(positions, torch.int32),
                              dev(token_seq, torch.int32), dev(table, torch.int32), heads,
                              kv_heads, head_dim, scale, window)
    qh = host(q).reshape(T, heads, head_dim)
    for t in range(T):
        s = token_seq[t]
        length = positions[t] + 1
        # blocks that fell out of a window may be gone (-1); they are never read
        first = max(0, positions[t] - window + 1) if window else 0
        kk = np.zeros((length, kv_heads, head_dim))
        vv = np.zeros((length, kv_heads, head_dim))
        kc, vc = host(k_cache), host(v_cache)
        for p in range(first, length):
            kk[p] = kc[table[s, p // 64], :, p % 64]
            vv[p] = vc[table[s, p // 64], :, p % 64]
        want = attention_reference(qh[t], kk, vv, positions[t], heads, kv_heads, scale, window)
        np.testing.assert_allclose(host(got[t]).reshape(heads, head_dim), want, rtol=0,
                                   atol=(2e-6 if dtype == torch.float32 else 8e-3),
                                   err_msg=f"token {t} at position {positions[t]}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """Every key is noise but one, far back in another block, which the query
    matches strongly: the output must be that key's value. A wrong block, a wrong
    offset or a wrong KV head shows at once."""
    rng = np.random.default_rng(5)
    heads, kv_heads, d = 6, 3, 64
    k_cache, v_cache = make_cache(rng, 10, kv_heads, d, dtype)
    k_cache *= 0.1
    table = np.array([[7, 1, 9, 3, 5, 0, 2, 8]], dtype=np.int32)
    pos = 500
    direction = rng.standard_normal(d)
    direction /= np.linalg.norm(direction)
    for far in (0, 63, 64, 257, 499, 500):
        kc = k_cache.clone()
        g = 1
        kc[table[0, far // 64], g, far % 64] = dev(direction * 40.0, dtype)
        q = np.zeros((1, heads, d))
        q[0, 2] = direction * 40.0             # head 2 and 3 read KV head 1
        q[0, 3] = direction * 40.0
        got = ops.attention_plain(dev(q.reshape(1, -1), dtype), kc, v_cache,
                                  dev([pos], torch.int32), dev([0], torch.int32),
                                  dev(table, torch.int32), heads, kv_heads, d, d ** -0.5, None)
        want = host(v_cache)[table[0, far // 64], g, far % 64]
        for h in (2, 3):
            np.testing.assert_allclose(host(got)[0, h * d:(h + 1) * d], want, rtol=0, atol=2e-2,
                                       err_msg=f"far key at {far}, head {h}")
        # a head of another group does not see it
        other = host(got)[0, 0:d]
        assert np.abs(other - want).max() > 0.1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_window_edge(dtype):
    """A towering key exactly at the window's edge is seen; one position further
    back it is not."""
    rng = np.random.default_rng(6)
    heads = kv_heads = 2
    d, window, pos = 32, 70, 200
    k_cache, v_cache = make_cache(rng, 4, kv_heads, d, dtype)
    k_cache *= 0.1
    table = np.array([[2, 0, 3, 1]], dtype=np.int32)
    direction = np.ones(d) / np.sqrt(d)
    q = np.tile(direction * 40.0, (1, heads))
    for far, seen in ((pos - window + 1, True), (pos - window, False)):
        kc = k_cache.clone()
        kc[table[0, far // 64], :, far % 64] = dev(np.tile(direction * 40.0, (kv_heads, 1)), dtype)
        got = ops.attention_plain(dev(q, dtype), kc, v_cache, dev([pos], torch.int32),
                                  dev([0], torch.int32), dev(table, torch.int32), heads, kv_heads,
                                  d, d ** -0.5, window)
        want = host(v_cache)[table[0, far // 64], 0, far % 64]
        close = np.abs(host(got)[0, :d] - want).max() < 2e-2
        assert close == seen, f"key at {far} (window {window}, query at {pos})"


def test_attention_ignores_what_lies_beyond_the_sequence():
    """NaN in every cache place after the query's position, and in blocks of other
    sequences, changes nothing."""
    rng = np.random.default_rng(7)
    heads, kv_heads, d = 4, 2, 16
    k_cache, v_cache = make_cache(rng, 6, kv_heads, d, torch.float32)
    table = np.array([[4, 1, -1]], dtype=np.int32)
    q = dev(rng.standard_normal((1, heads * d)))
    args = (dev([70], torch.int32), dev([0], torch.int32), dev(table, torch.int32), heads,
            kv_heads, d, 0.25, None)
    clean = ops.attention_plain(q, k_cache, v_cache, *args)
    for c in (k_cache, v_cache):
        c[1, :, 7:] = float("nan")              # positions 71.. of the sequence
        c[[0, 2, 3, 5]] = float("nan")          # other sequences' blocks
    dirty = ops.attention_plain(q, k_cache, v_cache, *args)
    assert torch.equal(clean, dirty)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_silu(dtype):
    rng = np.random.default_rng(8)
    gate = np.concatenate([rng.standard_normal((5, 171)) * 4, [[-100.0] * 171], [[90.0] * 171]])
    up = rng.standard_normal((7, 171))
    got = ops.gated_silu(dev(np.concatenate([gate, up], axis=1), dtype))
    g, u = host(dev(gate, dtype)), host(dev(up, dtype))
    want = g / (1 + np.exp(-g)) * u
    np.testing.assert_allclose(host(got), want, rtol=2 * ULP[dtype], atol=1e-30)
    assert np.isfinite(host(got)).all()
    # gate and up are not interchangeable
    swapped = ops.gated_silu(dev(np.concatenate([up, gate], axis=1), dtype))
    assert not torch.equal(swapped, got)


@pytest.mark.parametrize("M,N,K", [(1, 70, 33), (17, 64, 16), (65, 130, 200), (3, 1000, 352),
                                   (130, 48, 1)])
def test_gemm_f32(M, N, K):
    rng = np.random.default_rng(M * N + K)
    x, w, b = rng.standard_normal((M, K)), rng.standard_normal((N, K)), rng.standard_normal(N)
    xd, wd, bd = dev(x), dev(w), dev(b)
    want = host(xd) @ host(wd).T
    bound = 4 * np.sqrt(K) * 2.0 ** -24 * (np.abs(host(xd)) @ np.abs(host(wd)).T).max()
    got = ops.linear(xd, wd)
    assert np.abs(host(got) - want).max() <= bound
    got_b = ops.linear(xd, wd, bd)
    assert np.abs(host(got_b) - (want + host(bd))).max() <= bound + 1e-6
    acc = dev(rng.standard_normal((M, N)))
    before = host(acc)
    assert ops.linear(xd, wd, accumulate_into=acc) is acc
    assert np.abs(host(acc) - (before + want)).max() <= bound + 1e-6
    # a row's result does not depend on which other rows are in the batch
    for r in {0, M // 2, M - 1}:
        alone = ops.linear(xd[r:r + 1], wd)
        assert torch.equal(alone[0], got[r])


@pytest.mark.parametrize("M,N,K", [(1, 96, 64), (40, 200, 136), (300, 72, 1000)])
def test_linear_bf16(M, N, K):
    rng = np.random.default_rng(M + N + K)
    xd, wd = dev(rng.standard_normal((M, K)), torch.bfloat16), dev(rng.standard_normal((N, K)),
                                                                  torch.bfloat16)
    bd = dev(rng.standard_normal(N), torch.bfloat16)
    want = host(xd) @ host(wd).T
    scale = np.abs(want).max()
    got32 = ops.linear(xd, wd, out_dtype=torch.float32)
    assert got32.dtype == torch.float32
    assert np.abs(host(got32) - want).max() <= 1e-5 * scale * np.sqrt(K)
    got = ops.linear(xd, wd, bd)
    assert got.dtype == torch.bfloat16
    assert np.abs(host(got) - (want + host(bd))).max() <= 2.0 ** -8 * (scale + 4)
    acc = dev(rng.standard_normal((M, N)))
    before = host(acc)
    ops.linear(xd, wd, accumulate_into=acc)
    assert np.abs(host(acc) - (before + want)).max() <= 1e-5 * scale * np.sqrt(K) + 1e-6


def test_choose_greedy_rules():
    rows = np.array([[1.0, 3.0, 3.0, 2.0], [np.nan, 0.5, np.nan, 0.1],
                     [np.nan, np.nan, np.nan, np.nan], [-np.inf, -np.inf, -5.0, -np.inf]])
    got = ops.choose(dev(rows)).cpu().tolist()
    assert got == [1, 1, 4, 2]                  # 4 = past the end: no winner
    rng = np.random.default_rng(9)
    big = rng.standard_normal((5, 151937)).astype(np.float32)
    big[2, 77] = big[2, 150000] = 9.0           # a tie far apart: the lower index
    got = ops.choose(dev(big)).cpu().tolist()
    assert got == [plain.greedy(r) for r in big] and got[2] == 77


def test_choose_temperature_matches_plain_sampler():
    rng = np.random.default_rng(10)
    logits = (rng.standard_normal((6, 1000)) * 2).astype(np.float32)
    request = np.array([0, 1, 2, 3, 40, 7], dtype=np.int32)
    step = np.array([0, 5, 1, 1000, 3, 3], dtype=np.int32)
    got = ops.choose(dev(logits), 0.7, 99, dev(request, torch.int32), dev(step, torch.int32))
    want = [plain.sample(logits[i], 0.7, 99, int(request[i]), int(step[i])) for i in range(6)]
    assert got.cpu().tolist() == want
    # the row's place in the batch does not matter
    again = ops.choose(dev(logits[[4]]), 0.7, 99, dev(request[[4]], torch.int32),
                       dev(step[[4]], torch.int32))
    assert again.cpu().tolist() == [want[4]]


def test_kernels_refuse_what_they_cannot_take():
    with pytest.raises(ops.KernelError, match="CUDA device only"):
        ops.embed(torch.zeros(3, dtype=torch.int32), torch.zeros(4, 4))
    x = torch.zeros((2, 8), device=DEV)
    with pytest.raises(ops.KernelError):
        ops.rms_norm(x, torch.zeros(9, device=DEV), 1e-6, torch.float32)
    with pytest.raises(ops.KernelError, match="float32 or bfloat16"):
        ops.gated_silu(torch.zeros((2, 8), device=DEV, dtype=torch.float16))
    with pytest.raises(ops.KernelError, match="256"):
        ops.attention_plain(torch.zeros((1, 512), device=DEV),
                            torch.zeros((1, 1, 64, 512), device=DEV),
                            torch.zeros((1, 1, 64, 512), device=DEV),
                            torch.zeros(1, dtype=torch.int32, device=DEV),
                            torch.zeros(1, dtype=torch.int32, device=DEV),
                            torch.zeros((1, 1), dtype=torch.int32, device=DEV), 1, 1, 512, 1.0, None)


# ---- the bfloat16 tensor-core attention kernels ------------------------------------------

def paged_case(rng, lengths, kv_heads, d, n_blocks=64, poison=True):
    """A cache with scattered blocks for sequences of the given lengths. Blocks that no
    sequence holds, and the places past each sequence's end, are NaN."""
    k = rng.standard_normal((n_blocks, kv_heads, 64, d))
    v = rng.standard_normal((n_blocks, kv_heads, 64, d))
    order = rng.permutation(n_blocks)
    width = max(-(-n // 64) for n in lengths)
    table = np.full((len(lengths), width), -1, dtype=np.int32)
    used = np.zeros((n_blocks, 64), dtype=bool)
    at = 0
    for i, n in enumerate(lengths):
        for b in range(-(-n // 64)):
            table[i, b] = order[at]
            used[order[at], :min(64, n - 64 * b)] = True
            at += 1
    assert at <= n_blocks
    if poison:                       # `used` is [block, place]: spread it over the heads
        k.transpose(0, 2, 1, 3)[~used] = np.nan
        v.transpose(0, 2, 1, 3)[~used] = np.nan
    return dev(k, torch.bfloat16), dev(v, torch.bfloat16), table


def sequence_kv(cache, table_row, length):
    c = host(cache)
    out = np.zeros((length,) + c.shape[1:2] + c.shape[3:])
    for p in range(length):
        out[p] = c[table_row[p // 64], :, p % 64]
    return out


@pytest.mark.parametrize("heads,kv_heads,d,window", [(12, 2, 128, None), (4, 4, 64, None),
                                                     (16, 1, 128, None), (6, 3, 64, 100),
                                                     (14, 2, 128, 64), (5, 5, 128, 1)])
@pytest.mark.parametrize("splits", [1, 3, 20, 33, 64, None])      # 20 and more: the fold in groups
def test_attention_decode_kernel(heads, kv_heads, d, window, splits):
    rng = np.random.default_rng(heads * d + (window or 0))
    lengths = [1, 63, 64, 65, 700, 2048, 129]
    k_cache, v_cache, table = paged_case(rng, lengths, kv_heads, d)
    if window:          # blocks wholly before the window may be gone
        for i, n in enumerate(lengths):
            table[i, :max(0, n - window) // 64] = -1
    B = len(lengths)
    width = (heads + 2 * kv_heads) * d
    qkv = dev(rng.standard_normal((B, width)), torch.bfloat16)
    scale = d ** -0.5
    got = ops.attention_decode(qkv, k_cache, v_cache, dev(lengths, torch.int32),
                               dev(table, torch.int32), heads, kv_heads, d, scale, window,
                               max(lengths), splits=splits)
    assert all(v == 0 for v in ops.kernel_errors().values())
    q = host(qkv)[:, :heads * d].reshape(B, heads, d)
    for i, n in enumerate(lengths):
        first = max(0, n - window) if window else 0
        kk, vv = np.zeros((n, kv_heads, d)), np.zeros((n, kv_heads, d))
        kc, vc = host(k_cache), host(v_cache)
        for p in range(first, n):
            kk[p], vv[p] = kc[table[i, p // 64], :, p % 64], vc[table[i, p // 64], :, p % 64]
        want = attention_reference(q[i], kk, vv, n - 1, heads, kv_heads, scale, window)
        np.testing.assert_allclose(host(got[i]).reshape(heads, d), want, rtol=0, atol=1.5e-2,
                                   err_msg=f"sequence {i} of length {n}")
    # the plain kernel agrees too (same inputs, same cache)
    pos = dev([n - 1 for n in lengths], torch.int32)
    plain_out = ops.attention_plain(qkv, k_cache, v_cache, pos, dev(np.arange(B), torch.int32),
                                    dev(table, torch.int32), heads, kv_heads, d, scale, window)
    np.testing.assert_allclose(host(got), host(plain_out), rtol=0, atol=2e-2)


@pytest.mark.parametrize("heads,kv_heads,d,window", [(12, 2, 128, None), (4, 4, 64, None),
                                                     (16, 1, 128, None), (6, 3, 64, 100),
                                                     (14, 2, 128, 64)])
@pytest.mark.parametrize("splits", [2, 3, 4, 7, 8, 16])
@pytest.mark.parametrize("rotary", [False, True])
def test_attention_decode_folds_its_splits_as_a_cluster(heads, kv_heads, d, window, splits, rotary):
    """The splits of a (sequence, KV head) as one thread-block cluster that folds its partials
    through distributed shared memory (what the step uses for 2 and 4 splits): the float64
    reference's output, the second-kernel path's to a rounding of the fold's sums, the same
    cache afterwards; sequences with fewer key tiles than splits (blocks with no key) and
    lengths the kernel cannot serve among them."""
    rng = np.random.default_rng(heads * d + (window or 0) + splits)
    lengths = [1, 63, 64, 65, 700, 2048, 129, 0]
    k_cache, v_cache, table = paged_case(rng, [max(n, 1) for n in lengths], kv_heads, d)
    if window:
        for i, n in enumerate(lengths):
            table[i, :max(0, n - window) // 64] = -1
    B = len(lengths)
    qkv = dev(rng.standard_normal((B, (heads + 2 * kv_heads) * d)), torch.bfloat16)
    j = np.arange(d // 2)
    angle = np.arange(2304)[:, None] * np.power(1e4, -2.0 * j / d)[None, :]
    tables = (dev(np.cos(angle)), dev(np.sin(angle))) if rotary else None
    lens, tab = dev(lengths, torch.int32), dev(table, torch.int32)
    scale = d ** -0.5
    assert splits <= ops.attention.fold_cluster_limit(d)
    caches = [(k_cache.clone(), v_cache.clone()) for _ in range(2)]
    got, want = (ops.attention_decode(qkv, kc, vc, lens, tab, heads, kv_heads, d, scale, window,
                                      max(lengths), splits=splits, rotary=tables, in_cluster=way)
                 for way, (kc, vc) in zip((True, False), caches))
    assert all(v == 0 for v in ops.kernel_errors().values())
    assert torch.isfinite(got.float()).all() and torch.count_nonzero(got[-1]) == 0
    np.testing.assert_allclose(host(got), host(want), rtol=0, atol=2.0 ** -7)
    for a, b in zip(caches[0], caches[1]):
        np.testing.assert_array_equal(host(a), host(b))          # (NaN in unused blocks)
    if not rotary:
        q = host(qkv)[:, :heads * d].reshape(B, heads, d)
        for i, n in enumerate(lengths[:-1]):
            first = max(0, n - window) if window else 0
            kk, vv = np.zeros((n, kv_heads, d)), np.zeros((n, kv_heads, d))
            kc, vc = host(k_cache), host(v_cache)
            for p_ in range(first, n):
                kk[p_], vv[p_] = kc[table[i, p_ // 64], :, p_ % 64], vc[table[i, p_ // 64], :, p_ % 64]
            ref = attention_reference(q[i], kk, vv, n - 1, heads, kv_heads, scale, window)
            np.testing.assert_allclose(host(got[i]).reshape(heads, d), ref, rtol=0, atol=1.5e-2,
                                       err_msg=f"sequence {i} of length {n}")


def test_attention_decode_refuses_a_cluster_it_cannot_launch():
    rng = np.random.default_rng(3)
    k_cache, v_cache, table = paged_case(rng, [200], 1, 64)
    qkv = dev(rng.standard_normal((1, 4 * 64)), torch.bfloat16)
    with pytest.raises(ops.KernelError, match="do not fold as one cluster"):
        ops.attention_decode(qkv, k_cache, v_cache, dev([200], torch.int32), dev(table, torch.int32),
                             2, 1, 64, 0.125, None, 200, splits=17, in_cluster=True)


@pytest.mark.parametrize("splits", [None, 1, 7, 64])
def test_attention_decode_at_the_long_contexts_of_the_benchmark(splits):
    """16,385 and 32,352 cached positions (block lists of more than 500 blocks, more key tiles
    in a split than the kernel lists in shared memory) beside a short sequence."""
    heads, kv_heads, d = 12, 2, 128
    rng = np.random.default_rng(77)
    lengths = [16385, 70, 32352]
    k_cache, v_cache, table = paged_case(rng, lengths, kv_heads, d, n_blocks=768)
    B = len(lengths)
    qkv = dev(rng.standard_normal((B, (heads + 2 * kv_heads) * d)), torch.bfloat16)
    scale = d ** -0.5
    # Among thousands of random keys every output is near zero and a lost run of keys would
    # not show: three keys of each sequence (near its start, in its middle, next to its end)
    # are made to score 12 against the first query head of their KV head, so that they carry
    # most of that head's weight and the crowd of the others a tenth of it.
    group = heads // kv_heads
    for i, n in enumerate(lengths):
        for g in range(kv_heads):
            query = qkv[i, g * group * d:(g * group + 1) * d].float()
            planted = (query * (12.0 / (scale * float(query.norm()) ** 2))).to(torch.bfloat16)
            for p_ in (5, n // 2, n - 2):
                k_cache[int(table[i, p_ // 64]), g, p_ % 64] = planted
    got = ops.attention_decode(qkv, k_cache, v_cache, dev(lengths, torch.int32),
                               dev(table, torch.int32), heads, kv_heads, d, scale, None,
                               max(lengths), splits=splits)
    assert all(v == 0 for v in ops.kernel_errors().values())
    q = host(qkv)[:, :heads * d].reshape(B, heads, d)
    for i, n in enumerate(lengths):
        kk, vv = sequence_kv(k_cache, table[i], n), sequence_kv(v_cache, table[i], n)
        want = attention_reference(q[i], kk, vv, n - 1, heads, kv_heads, scale, None)
        np.testing.assert_allclose(host(got[i]).reshape(heads, d), want, rtol=0, atol=1.5e-2,
                                   err_msg=f"sequence of length {n}")


@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("rotary", [False, True])
def test_attention_decode_with_lengths_it_cannot_serve(splits, rotary):
    """A sequence whose length is 0, negative or beyond its block list (the engine never
    passes one; a caller of the exported function might) gets zeros, reads nothing outside
    the tables and writes nothing into the cache; its neighbours in the batch are served."""
    heads, kv_heads, d = 4, 2, 64
    rng = np.random.default_rng(9)
    good = [70, 1, 200]
    k_cache, v_cache, table = paged_case(rng, good + [64, 64, 64], kv_heads, d)
    lengths = good + [0, -5, table.shape[1] * 64 + 1]
    B = len(lengths)
    qkv = dev(rng.standard_normal((B, (heads + 2 * kv_heads) * d)), torch.bfloat16)
    j = np.arange(d // 2)
    angle = np.arange(256)[:, None] * np.power(1e4, -2.0 * j / d)[None, :]
    tables = (dev(np.cos(angle)), dev(np.sin(angle))) if rotary else None
    k_before, v_before = k_cache.clone(), v_cache.clone()
    lens, tab = dev(lengths, torch.int32), dev(table, torch.int32)
    got = ops.attention_decode(qkv, k_cache, v_cache, lens, tab, heads, kv_heads, d, d ** -0.5,
                               None, 256, splits=splits, rotary=tables)
    assert all(v == 0 for v in ops.kernel_errors().values())
    assert torch.count_nonzero(got[len(good):]) == 0 and torch.isfinite(got.float()).all()
    want = ops.attention_decode(qkv[:3].contiguous(), k_before.clone(), v_before.clone(), lens[:3].contiguous(),
                                tab[:3].contiguous(), heads, kv_heads, d, d ** -0.5, None, 256,
                                splits=splits, rotary=tables)
    assert torch.equal(got[:3], want)
    for now, was, blocks in ((k_cache, k_before, table), (v_cache, v_before, table)):
        for i in range(len(good), B):          # the blocks of the unserved sequences: untouched
            mine = torch.as_tensor(blocks[i][blocks[i] >= 0], device=DEV, dtype=torch.long)
            a, b = now[mine], was[mine]
            assert torch.equal(torch.nan_to_num(a.float()), torch.nan_to_num(b.float()))


@pytest.mark.parametrize("heads,kv_heads,d,window,splits", [
    (12, 2, 128, None, None), (12, 2, 128, None, 1), (2, 1, 64, None, 3), (6, 6, 64, 70, None),
    (7, 1, 128, 200, 5), (16, 1, 128, None, 2)])
def test_attention_decode_rotates_and_stores_on_its_way(heads, kv_heads, d, window, splits):
    """With rotary tables the decode kernel takes the projection's output as it came: what it
    returns, and what it leaves in the cache, is what the position kernel followed by the
    decode kernel gives; with `write_cache=False` the cache is only read."""
    rng = np.random.default_rng(heads * d + (window or 0))
    lengths = [1, 63, 64, 65, 700, 2048, 129, 128]
    k_cache, v_cache, table = paged_case(rng, lengths, kv_heads, d)
    if window:
        for i, n in enumerate(lengths):
            table[i, :max(0, n - window) // 64] = -1
    B = len(lengths)
    width = (heads + 2 * kv_heads) * d
    qkv = dev(rng.standard_normal((B, width)), torch.bfloat16)
    j = np.arange(d // 2)
    angle = np.arange(2304)[:, None] * np.power(1e4, -2.0 * j / d)[None, :]
    cos, sin = dev(np.cos(angle)), dev(np.sin(angle))
    lens, tab = dev(lengths, torch.int32), dev(table, torch.int32)
    scale = d ** -0.5
    # the two kernels, one after the other
    k_two, v_two, q_two = k_cache.clone(), v_cache.clone(), qkv.clone()
    ops.rope_store(q_two, dev([n - 1 for n in lengths], torch.int32), dev(np.arange(B), torch.int32),
                   tab, cos, sin, k_two, v_two, heads, kv_heads, d)
    want = ops.attention_decode(q_two, k_two, v_two, lens, tab, heads, kv_heads, d, scale, window,
                                max(lengths), splits=splits)
    # the one kernel
    k_one, v_one = k_cache.clone(), v_cache.clone()
    got = ops.attention_decode(qkv, k_one, v_one, lens, tab, heads, kv_heads, d, scale, window,
                               max(lengths), splits=splits, rotary=(cos, sin))
    assert all(v == 0 for v in ops.kernel_errors().values())
    np.testing.assert_allclose(host(got), host(want), rtol=0, atol=4e-3)
    np.testing.assert_allclose(host(k_one), host(k_two), rtol=0, atol=2.0 ** -6)
    np.testing.assert_array_equal(host(v_one), host(v_two))       # (NaN in unused blocks)
    for now, was in ((k_one, k_cache), (v_one, v_cache)):
        a, b = host(now), host(was)
        changed = ((a != b) & ~(np.isnan(a) & np.isnan(b))).any(axis=(1, 3))     # [block, row]
        assert changed.sum() <= B
    # a layer that reads another layer's cache: the newest key is there already
    k_read, v_read = k_two.clone(), v_two.clone()
    again = ops.attention_decode(qkv, k_read, v_read, lens, tab, heads, kv_heads, d, scale, window,
                                 max(lengths), splits=splits, rotary=(cos, sin), write_cache=False)
    np.testing.assert_allclose(host(again), host(want), rtol=0, atol=4e-3)
    np.testing.assert_array_equal(host(k_read), host(k_two))
    np.testing.assert_array_equal(host(v_read), host(v_two))


@pytest.mark.parametrize("heads,kv_heads,d,window", [(12, 2, 128, None), (2, 1, 64, None),
                                                     (6, 6, 64, 70), (7, 1, 128, 200)])
def test_attention_prefill_kernel(heads, kv_heads, d, window):
    rng = np.random.default_rng(heads + d + (window or 0))
    # (cached before the step, new tokens): whole prompts, one that ends on a block's
    # edge, a chunk that continues a long prefix, single tokens
    cases = [(0, 150), (0, 64), (299, 1), (64, 2), (100, 130), (0, 1), (37, 91), (600, 200)]
    lengths = [a + n for a, n in cases]
    k_cache, v_cache, table = paged_case(rng, lengths, kv_heads, d)
    T = sum(n for _, n in cases)
    width = (heads + 2 * kv_heads) * d
    qkv = dev(rng.standard_normal((T, width)), torch.bfloat16)
    tiles, row = [], 0
    for i, (a, n) in enumerate(cases):
        for s in range(0, n, 64):
            tiles.append((i, row + s, min(64, n - s), a + s))
        row += n
    scale = d ** -0.5
    got = ops.attention_prefill(qkv, k_cache, v_cache, dev(tiles, torch.int32),
                                dev(lengths, torch.int32), dev(table, torch.int32), heads,
                                kv_heads, d, scale, window)
    assert ops.kernel_errors()["sakv_prefill_attention_error"] == 0
    q = host(qkv)[:, :heads * d].reshape(T, heads, d)
    row = 0
    for i, (a, n) in enumerate(cases):
        kk = sequence_kv(k_cache, table[i], lengths[i])
        vv = sequence_kv(v_cache, table[i], lengths[i])
        for t in range(n):
            want = attention_reference(q[row + t], kk, vv, a + t, heads, kv_heads, scale, window)
            np.testing.assert_allclose(host(got[row + t]).reshape(heads, d), want, rtol=0,
                                       atol=1.5e-2, err_msg=f"case {i}, token {t}")
        row += n


@pytest.mark.parametrize("kernel", ["decode", "prefill"])
def test_tensor_core_attention_finds_one_far_key(kernel):
    rng = np.random.default_rng(11)
    heads, kv_heads, d = 12, 2, 128
    n = 1500
    k_cache, v_cache, table = paged_case(rng, [n], kv_heads, d, n_blocks=32)
    k_cache *= 0.05
    direction = rng.standard_normal(d)
    direction /= np.linalg.norm(direction)
    for far in (0, 63, 64, 777, 1471, 1472, 1499):
        kc = k_cache.clone()
        kc[table[0, far // 64], 1, far % 64] = dev(direction * 60.0, torch.bfloat16)
        q = np.zeros((1, heads + 2 * kv_heads, d))
        q[0, 6:12] = direction * 60.0                     # the heads of KV head 1
        qkv = dev(q.reshape(1, -1), torch.bfloat16)
        if kernel == "decode":
            got = ops.attention_decode(qkv, kc, v_cache, dev([n], torch.int32),
                                       dev(table, torch.int32), heads, kv_heads, d, d ** -0.5,
                                       None, n)
        else:
            got = ops.attention_prefill(qkv, kc, v_cache, dev([(0, 0, 1, n - 1)], torch.int32),
                                        dev([n], torch.int32), dev(table, torch.int32), heads,
                                        kv_heads, d, d ** -0.5, None)
        want = host(v_cache)[table[0, far // 64], 1, far % 64]
        out = host(got).reshape(heads, d)
        for h in range(6, 12):
            np.testing.assert_allclose(out[h], want, rtol=0, atol=2e-2,
                                       err_msg=f"{kernel}: far key at {far}, head {h}")
        assert np.abs(out[0] - want).max() > 0.1


# ---- the tcgen05 matrix product -----------------------------------------------------------

@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 1536, 1536), (8, 2048, 1536), (16, 70, 72),
                                   (17, 1000, 352), (64, 1536, 8960), (100, 384, 200),
                                   (256, 640, 1536), (3, 151936 // 8, 256),
                                   (20, 19200, 1536), (40, 19200, 1536)])   # many waves, odd rings
@pytest.mark.parametrize("splits", [None, 1, 3, 8])
def test_gemm_tc_epilogues(M, N, K, splits):
    from semantic_aware_adaptive_kv_cache_precision_b200.ops import gemm_tc
    rng = np.random.default_rng(M + N + K)
    x = dev(rng.standard_normal((M, K)), torch.bfloat16)
    w = dev(rng.standard_normal((N, K)), torch.bfloat16)
    b = dev(rng.standard_normal(N), torch.bfloat16)
    assert gemm_tc.takes(x, w)
    want = host(x) @ host(w).T
    scale = np.abs(want).max()
    out32 = torch.empty((M, N), dtype=torch.float32, device=DEV)
    gemm_tc.gemm(x, w, None, gemm_tc.EPI_F32, out32, N, splits=splits)
    assert gemm_tc.error_word() == 0
    assert np.abs(host(out32) - want).max() <= 2e-6 * scale * np.sqrt(K) + 1e-6
    out16 = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm(x, w, b, gemm_tc.EPI_BF16, out16, N, splits=splits)
    assert np.abs(host(out16) - (want + host(b))).max() <= 2.0 ** -8 * (scale + 4)
    acc = dev(rng.standard_normal((M, N)))
    before = host(acc)
    gemm_tc.gemm(x, w, None, gemm_tc.EPI_ACCUM, acc, N, splits=splits)
    gemm_tc.gemm(x, w, None, gemm_tc.EPI_ACCUM, acc, N, splits=splits)      # tickets reset themselves
    assert np.abs(host(acc) - (before + 2 * want)).max() <= 4e-6 * scale * np.sqrt(K) + 1e-5
    assert gemm_tc.error_word() == 0


@pytest.mark.parametrize("M,N,K,parts,splits", [
    (8, 1536, 8960, 12, 1), (8, 1536, 1536, 12, 1), (64, 1536, 8960, 6, 2), (3, 200, 328, 3, 2),
    (17, 130, 2048, 16, 1), (1, 128, 128, 2, 1)])
def test_gemm_tc_k_ranges_summed_apart(M, N, K, parts, splits):
    """K cut into ranges whose sums are left apart: the bias is in the first, their sum is
    the product, and the norm that adds them on its way gives what the separate steps give."""
    from semantic_aware_adaptive_kv_cache_precision_b200.ops import gemm_tc
    rng = np.random.default_rng(M + N + K)
    x = dev(rng.standard_normal((M, K)), torch.bfloat16)
    w = dev(rng.standard_normal((N, K)), torch.bfloat16)
    b = dev(rng.standard_normal(N), torch.bfloat16)
    sums = torch.full((parts, M, N), float("nan"), dtype=torch.float32, device=DEV)
    gemm_tc.gemm(x, w, b, gemm_tc.EPI_F32, sums, N, splits=splits, parts=parts)
    assert gemm_tc.error_word() == 0
    want = host(x) @ host(w).T + host(b)
    got = host(sums)
    assert np.isfinite(got).all()
    assert np.abs(got.sum(0) - want).max() <= 2e-6 * np.abs(want).max() * np.sqrt(K) + 1e-6
    per = -(-(-(-K // 64)) // (parts * splits)) * 64 * splits         # columns of K per part
    for i in range(parts):
        part = host(x)[:, i * per:(i + 1) * per] @ host(w)[:, i * per:(i + 1) * per].T
        if i == 0:
            part = part + host(b)
        assert np.abs(got[i] - part).max() <= 2e-6 * np.abs(want).max() * np.sqrt(K) + 1e-6
    # the reader's side
    stream = dev(rng.standard_normal((M, N)))
    weight = dev(1 + 0.1 * rng.standard_normal(N), torch.bfloat16)
    apart = stream.clone()
    ops.add_into(apart, sums)
    want_normed = ops.rms_norm(apart, weight, 1e-5, torch.bfloat16)
    got_normed = ops.rms_norm(stream, weight, 1e-5, torch.bfloat16, add=sums)
    assert torch.equal(stream, apart) and torch.equal(got_normed, want_normed)


@pytest.mark.parametrize("kernel", ["pair", "single"])
@pytest.mark.parametrize("M,I,K", [(1030, 384, 1536), (256, 200, 72), (2048, 8960, 1536),
                                   (700, 128, 64), (513, 1096, 328), (65, 8, 8), (300, 18944, 136),
                                   (4200, 264, 3000)])
def test_gated_product_for_many_tokens(M, I, K, kernel):
    """The tcgen05 products with the gated SiLU in their epilogue (on pairs of SMs with
    `cta_group::2`, and on single blocks) against float64, and against the library's product
    followed by the activation kernel (a bf16 rounding apart): token counts that fill no
    tile, more tiles than pairs (several rounds through both accumulators), a K of one step and
    of 47, intermediate sizes that fill no tile of weight rows."""
    from semantic_aware_adaptive_kv_cache_precision_b200.ops import gemm_wide
    rng = np.random.default_rng(M + I + K)
    x = dev(rng.standard_normal((M, K)), torch.bfloat16)
    w = dev(rng.standard_normal((2 * I, K)) * (2.0 / np.sqrt(K)), torch.bfloat16)
    assert gemm_wide.takes(x, w)
    if kernel == "pair":
        assert gemm_wide.resident_pairs() > 0
        run, word = gemm_wide.gated_pair, gemm_wide.pair_error_word
    else:
        run, word = gemm_wide.gated, gemm_wide.error_word
    got = host(run(x, w))
    assert word() == 0
    both = host(x) @ host(w).T
    gate, up = both[:, :I], both[:, I:]
    want = gate / (1 + np.exp(-gate)) * up
    assert np.abs(got - want).max() <= 2.0 ** -8 * (np.abs(want).max() + 1) * 1.5
    twin = host(ops.gated_silu(torch.mm(x, w.t())))
    assert np.abs(got - twin).max() <= 2.0 ** -7 * (np.abs(want).max() + 1)
    assert torch.equal(run(x, w), run(x, w))                 # (the same sums every time)
    if kernel == "pair" and gemm_wide.pair_worth_it(M):
        assert torch.equal(ops.gated_up(x, w), gemm_wide.gated_pair(x, w))    # the product path takes it


def test_which_gated_product_runs():
    from semantic_aware_adaptive_kv_cache_precision_b200.ops import gemm_wide
    # on pairs: token tiles at least five eighths (one tile) or four fifths (several) full
    assert all(gemm_wide.pair_worth_it(t) for t in (160, 256, 410, 512, 768, 1024, 2048, 8192))
    assert not any(gemm_wide.pair_worth_it(t) for t in (1, 64, 65, 128, 159, 257, 384, 600))
    # single blocks (where no pair can be placed): whole waves of tiles, full token tiles
    assert gemm_wide.worth_it(2048, 8960, sms=148) and gemm_wide.worth_it(512, 8960, sms=148)
    assert gemm_wide.worth_it(256, 18944, sms=148)              # 148 tiles: one full wave
    assert not gemm_wide.worth_it(256, 8960, sms=148)           # 70 tiles: half a wave
    assert not gemm_wide.worth_it(768, 8960, sms=148)           # 210 tiles: 1.4 waves
    assert not gemm_wide.worth_it(300, 18944, sms=148)          # token tiles 59 % full
    assert not gemm_wide.worth_it(64, 18944, sms=148)


@pytest.mark.parametrize("T,N,K", [(2048, 1536, 8960), (100, 200, 136), (65, 1536, 1536), (300, 72, 64)])
def test_library_product_adds_into_the_stream_itself(T, N, K):
    """Above the own kernels' token count the product that completes an fp32 accumulator is
    cuBLAS with beta = 1 (`csrc/gemm_lib.cu`): the sum against float64, on an accumulator that
    is a view with a row stride of its own, and nothing handed back to be added later."""
    rng = np.random.default_rng(T + N + K)
    x = dev(rng.standard_normal((T, K)), torch.bfloat16)
    w = dev(rng.standard_normal((N, K)) / np.sqrt(K), torch.bfloat16)
    wide = dev(rng.standard_normal((T, N + 8)))
    acc = wide[:, :N]
    before, beside = host(acc), host(wide[:, N:])
    out = ops.linear(x, w, accumulate_into=acc, may_defer=True)
    assert out is acc
    want = before + host(x) @ host(w).T
    np.testing.assert_allclose(host(acc), want, rtol=0, atol=2e-5 * np.abs(want).max() + 1e-6)
    np.testing.assert_array_equal(host(wide[:, N:]), beside)        # nothing beside it is touched
    # with a bias the product still goes through torch and is handed back or added
    b = dev(rng.standard_normal(N), torch.bfloat16)
    acc2 = dev(before)
    out = ops.linear(x, w, b, accumulate_into=acc2)
    assert out is acc2
    np.testing.assert_allclose(host(acc2), want + host(b), rtol=0, atol=2e-5 * np.abs(want).max() + 1e-5)


def test_linear_hands_back_k_ranges_only_when_asked():
    rng = np.random.default_rng(5)
    x = dev(rng.standard_normal((8, 8960)), torch.bfloat16)
    w = dev(rng.standard_normal((1536, 8960)) * 0.02, torch.bfloat16)
    acc = dev(rng.standard_normal((8, 1536)))
    kept = acc.clone()
    out = ops.linear(x, w, accumulate_into=acc, may_defer=True)
    assert isinstance(out, ops.Deferred) and out.delta.dim() == 3 and torch.equal(acc, kept)
    same = ops.linear(x, w, accumulate_into=acc)
    assert same is acc
    want = host(kept) + host(x) @ host(w).T
    np.testing.assert_allclose(host(acc), want, rtol=0, atol=1e-4)
    ops.add_into(kept, out.delta)
    np.testing.assert_allclose(host(kept), want, rtol=0, atol=1e-4)
    # many row tiles: nothing to gain, the product is added where it is made
    wide = dev(rng.standard_normal((17920, 1536)) * 0.02, torch.bfloat16)
    acc2 = torch.zeros((8, 17920), device=DEV)
    assert ops.linear(dev(rng.standard_normal((8, 1536)), torch.bfloat16), wide,
                      accumulate_into=acc2, may_defer=True) is acc2


@pytest.mark.parametrize("M,I,K", [(1, 128, 64), (8, 8960, 1536), (50, 256, 200), (128, 384, 1536)])
def test_gemm_tc_gated(M, I, K):
    rng = np.random.default_rng(M + I + K)
    x = dev(rng.standard_normal((M, K)) * 0.5, torch.bfloat16)
    w = dev(rng.standard_normal((2 * I, K)) * 0.2, torch.bfloat16)
    got = ops.gated_up(x, w)
    assert got.shape == (M, I) and got.dtype == torch.bfloat16
    g = host(x) @ host(w[:I]).T
    u = host(x) @ host(w[I:]).T
    want = g / (1 + np.exp(-g)) * u
    assert np.abs(host(got) - want).max() <= 2.0 ** -7 * np.abs(want).max() + 1e-3
    two_step = ops.gated_silu(ops.linear(x, w, out_dtype=torch.bfloat16))
    assert np.abs(host(got) - host(two_step)).max() <= 2.0 ** -6 * np.abs(want).max() + 1e-3


def test_gemm_tc_long_k_loops_many_times():
    """Products whose blocks walk the ring of stages many times (56 and 60 K steps a block,
    as the 7B shape's), launched back to back: every launch gives the same bits, and they
    are right. (The two MMA lanes once shared stages of an odd ring; a lane that ran ahead
    then read a tile that had not landed.)"""
    rng = np.random.default_rng(11)
    M, H, I = 8, 3584, 18944
    x = dev(rng.standard_normal((M, H)) * 0.5, torch.bfloat16)
    w = dev(rng.standard_normal((2 * I, H)) * 0.05, torch.bfloat16)
    first = ops.gated_up(x, w)
    for _ in range(30):
        assert torch.equal(ops.gated_up(x, w), first)
    g = host(x) @ host(w[:I]).T
    u = host(x) @ host(w[I:]).T
    want = g / (1 + np.exp(-g)) * u
    assert np.abs(host(first) - want).max() <= 2.0 ** -7 * np.abs(want).max() + 1e-3
    xd = dev(rng.standard_normal((M, I)) * 0.5, torch.bfloat16)
    wd = dev(rng.standard_normal((H, I)) * 0.02, torch.bfloat16)
    sums = [ops.linear(xd, wd, out_dtype=torch.float32) for _ in range(30)]
    assert all(torch.equal(y, sums[0]) for y in sums)
    np.testing.assert_allclose(host(sums[0]), host(xd) @ host(wd).T, rtol=0, atol=2e-3)
    assert all(v == 0 for v in ops.kernel_errors().values())


def test_gemm_tc_refuses_what_it_cannot_take():
    from semantic_aware_adaptive_kv_cache_precision_b200.ops import gemm_tc
    x = torch.zeros((4, 36), dtype=torch.bfloat16, device=DEV)        # K not a multiple of 8
    w = torch.zeros((128, 36), dtype=torch.bfloat16, device=DEV)
    assert not gemm_tc.takes(x, w)
    out = ops.linear(x, w)                                            # the library product runs
    assert out.shape == (4, 128)
    assert not gemm_tc.takes(x.float(), w)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_vector_paths_of_the_elementwise_kernels(dtype):
    """Widths that are multiples of 8 take the 16-byte paths; they must agree with the
    scalar paths (odd widths) on the same values."""
    rng = np.random.default_rng(12)
    gate = rng.standard_normal((33, 176)) * 3
    up = rng.standard_normal((33, 176))
    wide = ops.gated_silu(dev(np.concatenate([gate, up], axis=1), dtype))
    narrow = ops.gated_silu(dev(np.concatenate([gate[:, :175], up[:, :175]], axis=1), dtype))
    assert torch.equal(wide[:, :175], narrow)
    acc = dev(rng.standard_normal((7, 64)))
    y = dev(rng.standard_normal((7, 64)), dtype)
    want = host(acc) + host(y)
    ops.add_into(acc, y)
    np.testing.assert_allclose(host(acc), want, rtol=0, atol=1e-6)


@pytest.mark.parametrize("slots", [296, 1])
def test_attention_prefill_tcgen05_kernel_after_a_long_prefix(slots):
    """A chunk of a prompt after 24,576 cached positions (a query tile walks 388 key tiles:
    the rings and their barrier phases wrap hundreds of times) beside one after 8,000, with
    three keys of each sequence planted to carry most of its last query's weight."""
    heads, kv_heads, d = 4, 2, 128
    rng = np.random.default_rng(slots)
    cases = [(24576, 200), (8000, 130)]
    lengths = [a + n for a, n in cases]
    k_cache, v_cache, table = paged_case(rng, lengths, kv_heads, d, n_blocks=560)
    T = sum(n for _, n in cases)
    qkv = dev(rng.standard_normal((T, (heads + 2 * kv_heads) * d)), torch.bfloat16)
    scale = d ** -0.5
    group = heads // kv_heads
    last_rows = [cases[0][1] - 1, T - 1]
    for i, (a, n) in enumerate(cases):
        for g in range(kv_heads):
            query = qkv[last_rows[i], g * group * d:(g * group + 1) * d].float()
            planted = (query * (12.0 / (scale * float(query.norm()) ** 2))).to(torch.bfloat16)
            for p_ in (3, a // 2 + 1, a + n - 2):
                k_cache[int(table[i, p_ // 64]), g, p_ % 64] = planted
    plan = ops.upload_wide_plan([a for a, _ in cases], [n for _, n in cases], heads, None, "cuda",
                                slots=slots)
    got = ops.attention_prefill_tc(qkv, k_cache, v_cache, *plan, dev(lengths, torch.int32),
                                   dev(table, torch.int32), heads, kv_heads, d, scale, None)
    assert ops.kernel_errors()["sakv_prefill_attention_tc_error"] == 0
    q = host(qkv)[:, :heads * d].reshape(T, heads, d)
    row = 0
    for i, (a, n) in enumerate(cases):
        kk = sequence_kv(k_cache, table[i], lengths[i])
        vv = sequence_kv(v_cache, table[i], lengths[i])
        for t in (0, 1, 63, 64, 127, 128, n - 2, n - 1):
            want = attention_reference(q[row + t], kk, vv, a + t, heads, kv_heads, scale, None)
            np.testing.assert_allclose(host(got[row + t]).reshape(heads, d), want, rtol=0,
                                       atol=1.5e-2, err_msg=f"case {i}, token {t}")
        assert np.abs(host(got[row + n - 1])).max() > 0.3        # the planted keys carry it
        row += n


# slots: how many blocks the plan believes run at once; 1 deals no tile to several blocks,
# a huge number cuts every tile of more than 8 key tiles
@pytest.mark.parametrize("heads,kv_heads,window,slots", [
    (12, 2, None, 296), (4, 4, None, 1), (4, 4, None, 10 ** 6), (7, 1, 200, 10 ** 6),
    (6, 3, 64, 296), (2, 1, 700, 10 ** 6)])
def test_attention_prefill_tcgen05_kernel(heads, kv_heads, window, slots):
    d = 128
    rng = np.random.default_rng(heads + (window or 0))
    cases = [(0, 150), (0, 128), (299, 1), (64, 2), (100, 130), (0, 1), (37, 91), (600, 300),
             (0, 1100)]
    lengths = [a + n for a, n in cases]
    k_cache, v_cache, table = paged_case(rng, lengths, kv_heads, d)
    T = sum(n for _, n in cases)
    width = (heads + 2 * kv_heads) * d
    qkv = dev(rng.standard_normal((T, width)), torch.bfloat16)
    plan = ops.upload_wide_plan([a for a, _ in cases], [n for _, n in cases], heads, window,
                                "cuda", slots=slots)
    assert slots > 1 or plan[1] is None
    scale = d ** -0.5
    got = ops.attention_prefill_tc(qkv, k_cache, v_cache, *plan,
                                   dev(lengths, torch.int32), dev(table, torch.int32), heads,
                                   kv_heads, d, scale, window)
    assert ops.kernel_errors()["sakv_prefill_attention_tc_error"] == 0
    q = host(qkv)[:, :heads * d].reshape(T, heads, d)
    row = 0
    for i, (a, n) in enumerate(cases):
        kk = sequence_kv(k_cache, table[i], lengths[i])
        vv = sequence_kv(v_cache, table[i], lengths[i])
        for t in range(n):
            want = attention_reference(q[row + t], kk, vv, a + t, heads, kv_heads, scale, window)
            np.testing.assert_allclose(host(got[row + t]).reshape(heads, d), want, rtol=0,
                                       atol=1.5e-2, err_msg=f"case {i}, token {t}")
        row += n
    # and its twin on the mma.sync path agrees
    tiles64, row = [], 0
    for i, (a, n) in enumerate(cases):
        for s in range(0, n, 64):
            tiles64.append((i, row + s, min(64, n - s), a + s))
        row += n
    twin = ops.attention_prefill(qkv, k_cache, v_cache, dev(tiles64, torch.int32),
                                 dev(lengths, torch.int32), dev(table, torch.int32), heads,
                                 kv_heads, d, scale, window)
    np.testing.assert_allclose(host(got), host(twin), rtol=0, atol=2e-2)
