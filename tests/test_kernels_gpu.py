"""Each CUDA kernel alone against its plain float64 reference, at sizes other than the engine's."""
import math

import pytest
import torch

from helpers import TOL, batch_index, paged_cache, rel_error
from plain import ops_plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from aegean_tge_b200 import ops as module
    module.core()
    return module


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab,hidden,tokens", [(97, 72, 13), (331, 200, 1)])
def test_embedding(ops, dtype, vocab, hidden, tokens):
    gen = torch.Generator().manual_seed(1)
    table = torch.randn(vocab, hidden, generator=gen).to(dtype)
    ids = torch.randint(0, vocab, (tokens,), generator=gen, dtype=torch.int32)
    out = ops.embedding(table.to(DEV), ids.to(DEV))
    assert out.dtype == torch.float32
    assert torch.equal(out.cpu(), table[ids.long()].float())
    ops.check_status()


def test_embedding_bad_token_is_reported_not_read(ops):
    table = torch.randn(10, 8).to(DEV)
    out = ops.embedding(table, torch.tensor([3, 10, -1], dtype=torch.int32, device=DEV))
    assert torch.equal(out[1:].cpu(), torch.zeros(2, 8))
    with pytest.raises(ops.DeviceStatusError):
        ops.check_status()
    ops.check_status()      # the word was cleared


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,hidden,eps", [(5, 72, 1e-6), (3, 200, 1e-5), (2, 3000, 3e-6), (1, 5120, 1e-6),
                                             (3, 70, 1e-6), (2, 9004, 1e-6), (300, 3584, 1e-6)])
def test_rmsnorm(ops, out_dtype, rows, hidden, eps):
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(rows, hidden, generator=gen) * 3.0
    w = 1.0 + (torch.rand(hidden, generator=gen) * 0.2 - 0.1)
    out = ops.rmsnorm(x.to(DEV), w.to(DEV), eps, out_dtype)
    assert rel_error(out, ops_plain.rmsnorm(x, w, eps)) < TOL[out_dtype]
    picked = torch.tensor([rows - 1, 0], dtype=torch.int32)
    out = ops.rmsnorm(x.to(DEV), w.to(DEV), eps, out_dtype, rows=picked.to(DEV))
    assert rel_error(out, ops_plain.rmsnorm(x[picked.long()], w, eps)) < TOL[out_dtype]
    ops.check_status()


def test_rmsnorm_eps_matters(ops):
    """Tiny inputs make eps dominate: a wrong or ignored eps shows at once."""
    x = torch.full((1, 64), 1e-4)
    w = torch.ones(64)
    for eps in (1e-6, 1e-5):
        out = ops.rmsnorm(x.to(DEV), w.to(DEV), eps, torch.float32)
        assert rel_error(out, ops_plain.rmsnorm(x, w, eps)) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_to_stream(ops, dtype):
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(7, 130, generator=gen)
    y = torch.randn(7, 130, generator=gen).to(dtype)
    dx = x.to(DEV)
    ops.add_to_stream(dx, y.to(DEV))
    assert torch.equal(dx.cpu(), x + y.float())


# ---------------------------------------------------------------------------
# products
# ---------------------------------------------------------------------------
SIMT_SHAPES = [(1, 64, 64), (7, 130, 72), (33, 200, 176), (65, 97, 50), (128, 256, 255)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", SIMT_SHAPES)
def test_gemm_simt_epilogues(ops, dtype, M, N, K):
    gen = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K, generator=gen).to(dtype)
    w = (torch.randn(N, K, generator=gen) * 0.1).to(dtype)
    b = torch.randn(N, generator=gen)
    ref = ops_plain.linear(x, w, b)
    out = ops.linear(x.to(DEV), w.to(DEV), b.to(DEV), ops.GEMM_STORE, force_simt=True)
    assert out.dtype == dtype and rel_error(out, ref) < TOL[dtype]
    out = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_STORE_F32, force_simt=True)
    assert out.dtype == torch.float32 and rel_error(out, ops_plain.linear(x, w, None)) < 2e-5
    stream = torch.randn(M, N, generator=gen)
    d = stream.to(DEV)
    ops.linear(x.to(DEV), w.to(DEV), b.to(DEV), ops.GEMM_ADD_F32, out=d, force_simt=True)
    assert rel_error(d, stream.double() + ref) < 2e-5
    if N % 2 == 0:
        out = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_SWIGLU, force_simt=True)
        assert out.shape == (M, N // 2) and rel_error(out, ops_plain.swiglu_interleaved(x, w)) < TOL[dtype]


def test_gemm_simt_value_does_not_depend_on_the_batch(ops):
    """A row's float32 product is bit-identical alone and inside a larger batch."""
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(70, 200, generator=gen).to(DEV)
    w = torch.randn(150, 200, generator=gen).to(DEV)
    whole = ops.linear(x, w, None, ops.GEMM_STORE_F32, force_simt=True)
    for row in (0, 33, 69):
        alone = ops.linear(x[row:row + 1], w, None, ops.GEMM_STORE_F32, force_simt=True)
        assert torch.equal(alone[0], whole[row])


TC_SHAPES = [(1, 128, 64), (8, 384, 176), (16, 200, 256), (33, 130, 72), (64, 512, 1024), (100, 300, 512),
             (200, 640, 320), (300, 1024, 512), (520, 256, 192)]


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_gemm_tcgen05_exact_on_small_integers(ops, M, N, K):
    """Integer-valued operands make every product and sum exact in float32, so any misplaced
    row, column, k-block or swizzle shows as an outright mismatch."""
    gen = torch.Generator().manual_seed(M + N + K)
    x = torch.randint(-2, 3, (M, K), generator=gen).to(torch.bfloat16)
    w = torch.randint(-3, 4, (N, K), generator=gen).to(torch.bfloat16)
    ref = (x.double() @ w.double().T).float()
    out = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_STORE_F32)
    ops.check_status()
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("M,N,K,bn,splits", [
    (5, 256, 512, 16, 1), (5, 256, 512, 16, 4), (40, 384, 1024, 64, 3), (130, 200, 576, 128, 2),
    (260, 512, 256, 256, 1), (260, 512, 1024, 256, 2), (70, 130, 176, 32, 1), (24, 3584, 512, 32, 1),
    (500, 384, 640, 208, 1), (300, 256, 320, 144, 2), (100, 200, 256, 48, 1), (470, 130, 192, 240, 1)])
def test_gemm_tcgen05_tiles_and_splits(ops, M, N, K, bn, splits):
    gen = torch.Generator().manual_seed(bn + splits + M)
    x = torch.randint(-2, 3, (M, K), generator=gen).to(torch.bfloat16)
    w = torch.randint(-3, 4, (N, K), generator=gen).to(torch.bfloat16)
    ref = (x.double() @ w.double().T).float()
    out = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_STORE_F32, force_bn=bn, force_splits=splits)
    ops.check_status()
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("M,N,K,splits", [(9, 260, 328, 1), (9, 260, 328, 3), (150, 384, 704, 1), (2048, 512, 256, 1),
                                          (2048, 3584, 128, 1), (1100, 640, 192, 1)])
def test_gemm_tcgen05_epilogues(ops, M, N, K, splits):
    gen = torch.Generator().manual_seed(7 * M + splits)
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=gen) * 0.1).to(torch.bfloat16)
    b = torch.randn(N, generator=gen)
    ref = ops_plain.linear(x, w, b)
    kw = dict(force_splits=splits)
    out = ops.linear(x.to(DEV), w.to(DEV), b.to(DEV), ops.GEMM_STORE, **kw)
    assert out.dtype == torch.bfloat16 and rel_error(out, ref) < TOL[torch.bfloat16]
    out = ops.linear(x.to(DEV), w.to(DEV), b.to(DEV), ops.GEMM_STORE_F32, **kw)
    assert rel_error(out, ref) < 2e-5
    stream = torch.randn(M, N, generator=gen)
    d = stream.to(DEV)
    ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_ADD_F32, out=d, **kw)
    assert rel_error(d, stream.double() + ops_plain.linear(x, w, None)) < 2e-5
    out = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_SWIGLU, **kw)
    assert out.shape == (M, N // 2) and rel_error(out, ops_plain.swiglu_interleaved(x, w)) < TOL[torch.bfloat16]
    ops.check_status()


@pytest.fixture
def pair_everywhere(ops):
    """Every bfloat16 product that the two-SM kernel can run goes to it, also shapes it would not be chosen for."""
    ops.set_pair_gemm(2)
    yield
    ops.set_pair_gemm(1)


@pytest.mark.parametrize("M,N,K", TC_SHAPES + [(2048, 768, 192), (257, 130, 136), (140, 3584, 64), (1000, 520, 1032)])
def test_gemm_pair_exact_on_small_integers(ops, pair_everywhere, M, N, K):
    """The kernel that pairs two SMs on a tile of 256 weight rows: rows of either block, token halves of
    either block, ragged edges in both directions, more k-blocks than stages."""
    gen = torch.Generator().manual_seed(M + N + K)
    x = torch.randint(-2, 3, (M, K), generator=gen).to(torch.bfloat16)
    w = torch.randint(-3, 4, (N, K), generator=gen).to(torch.bfloat16)
    ref = (x.double() @ w.double().T).float()
    out = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_STORE_F32)
    ops.check_status()
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("M,N,K", [(9, 260, 328), (150, 384, 704), (2048, 512, 256), (1100, 640, 192)])
def test_gemm_pair_epilogues(ops, pair_everywhere, M, N, K):
    gen = torch.Generator().manual_seed(7 * M)
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=gen) * 0.1).to(torch.bfloat16)
    b = torch.randn(N, generator=gen)
    ref = ops_plain.linear(x, w, b)
    out = ops.linear(x.to(DEV), w.to(DEV), b.to(DEV), ops.GEMM_STORE)
    assert out.dtype == torch.bfloat16 and rel_error(out, ref) < TOL[torch.bfloat16]
    out = ops.linear(x.to(DEV), w.to(DEV), b.to(DEV), ops.GEMM_STORE_F32)
    assert rel_error(out, ref) < 2e-5
    stream = torch.randn(M, N, generator=gen)
    d = stream.to(DEV)
    ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_ADD_F32, out=d)
    assert rel_error(d, stream.double() + ops_plain.linear(x, w, None)) < 2e-5
    out = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_SWIGLU)
    assert out.shape == (M, N // 2) and rel_error(out, ops_plain.swiglu_interleaved(x, w)) < TOL[torch.bfloat16]
    ops.check_status()


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (8, 3584, 512), (33, 520, 264), (128, 1024, 320), (140, 384, 192), (150, 384, 192)])
@pytest.mark.parametrize("defer", [False, True])
def test_linear_add_norm_and_rows_without_their_factor(ops, M, N, K, defer):
    """stream += x . w^T; the next product's input = RMSNorm(stream) * weight, either complete or (up to 128
    rows, if asked) without the norm's factor, which the product that takes the rows then applies: with a bias,
    with the gated epilogue, cut along k or not, and completed on their own."""
    gen = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=gen) * 0.1).to(torch.bfloat16)
    stream = torch.randn(M, N, generator=gen) * 3.0
    gain = 1.0 + 0.2 * torch.randn(N, generator=gen)
    eps = 1e-5
    new_stream = stream.double() + ops_plain.linear(x, w, None)
    normed = ops_plain.rmsnorm(new_stream, gain, eps)
    d_stream = stream.to(DEV)
    rows = ops.linear_add_norm(x.to(DEV), w.to(DEV), None, d_stream, gain.to(DEV), eps, torch.bfloat16, defer=defer)
    assert rel_error(d_stream, new_stream) < 2e-5
    assert isinstance(rows, ops.DeferredRows) == (defer and M <= 128)
    if isinstance(rows, ops.DeferredRows):
        assert rel_error(rows.complete(), normed) < 2 * TOL[torch.bfloat16]
    else:
        assert rel_error(rows, normed) < TOL[torch.bfloat16]
    # takers: a plain product with a bias (few weight rows and a long k: cut along k) and a gated one
    for rows_out, k_cut in ((40, True), (768, False)):
        w2 = (torch.randn(rows_out, N, generator=gen) * 0.05).to(torch.bfloat16)
        b2 = torch.randn(rows_out, generator=gen)
        want = ops_plain.linear(normed, w2, b2)
        got = ops.linear(rows, w2.to(DEV), b2.to(DEV), ops.GEMM_STORE_F32)
        assert rel_error(got, want) < TOL[torch.bfloat16], (rows_out, k_cut)
        got = ops.linear(rows, w2.to(DEV), None, ops.GEMM_SWIGLU)
        assert rel_error(got, ops_plain.swiglu_interleaved(normed, w2)) < 2 * TOL[torch.bfloat16]
    ops.check_status()


def test_gemm_tcgen05_refuses_what_tma_cannot_address(ops):
    """K that is no multiple of 8 cannot be a TMA row pitch: the product still comes out right (CUDA cores)."""
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(5, 50, generator=gen).to(torch.bfloat16)
    w = torch.randn(24, 50, generator=gen).to(torch.bfloat16)
    out = ops.linear(x.to(DEV), w.to(DEV), None, ops.GEMM_STORE_F32)
    assert rel_error(out, ops_plain.linear(x, w, None)) < 2e-5


# ---------------------------------------------------------------------------
# rotation + cache store
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary", [(6, 2, 48, 48), (5, 1, 64, 32), (4, 4, 16, 16), (3, 1, 80, 0),
                                                          (2, 1, 20, 12), (28, 4, 128, 128), (3, 2, 36, 36)])
def test_rope_kv_store(ops, dtype, heads, kv_heads, head_dim, rotary):
    from aegean_tge_b200.parts.rope import rotary_tables
    page_size = 16
    q_lens, starts = [5, 1, 20], [30, 47, 0]          # portions crossing page edges at odd offsets
    positions, seq_of_token, _, _ = batch_index(q_lens, starts, DEV)
    T = sum(q_lens)
    width = (heads + 2 * kv_heads) * head_dim
    gen = torch.Generator().manual_seed(heads * 10 + head_dim)
    qkv = torch.randn(T, width, generator=gen).to(dtype)
    lengths = [s + n for s, n in zip(starts, q_lens)]
    k_pages, v_pages, table, _, _ = paged_cache(lengths, kv_heads, head_dim, page_size, dtype, DEV, seed=4)
    before_k = k_pages.clone()
    cos = sin = None
    if rotary:
        cos, sin = rotary_tables(12345.0, rotary, 64)
    dq = qkv.to(DEV)
    ops.rope_kv_store(dq, None if cos is None else cos.to(DEV), None if sin is None else sin.to(DEV), rotary,
                      positions, seq_of_token, table, k_pages, v_pages, heads, kv_heads, head_dim)
    ops.check_status()
    pos = positions.cpu().long()
    q = qkv[:, :heads * head_dim].view(T, heads, head_dim)
    k = qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].view(T, kv_heads, head_dim)
    v = qkv[:, (heads + kv_heads) * head_dim:].view(T, kv_heads, head_dim)
    c = cos[pos] if rotary else None
    s = sin[pos] if rotary else None
    q_ref = ops_plain.rotate_half(q, c, s, rotary)
    k_ref = ops_plain.rotate_half(k, c, s, rotary)
    assert rel_error(dq[:, :heads * head_dim].reshape(T, heads, head_dim), q_ref) < TOL[dtype]
    touched = torch.zeros_like(before_k, dtype=torch.bool)
    for t in range(T):
        page = int(table[int(seq_of_token[t]), int(pos[t]) // page_size])
        slot = int(pos[t]) % page_size
        assert rel_error(k_pages[page, :, slot], k_ref[t]) < TOL[dtype]
        assert torch.equal(v_pages[page, :, slot].cpu(), v[t])
        touched[page, :, slot] = True
    assert torch.equal(k_pages[~touched], before_k[~touched]), "a slot outside the step's positions was written"


@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary,hidden", [(7, 1, 128, 128, 512), (4, 2, 128, 0, 256), (6, 2, 64, 64, 384),
                                                                 (5, 1, 64, 32, 320)])
@pytest.mark.parametrize("q_lens,starts", [([1, 1, 1], [30, 47, 0]), ([5, 1, 20], [30, 47, 0]), ([70, 58], [3, 16]), ([80, 62], [3, 16]), ([90, 70], [3, 6])])
@pytest.mark.parametrize("deferred", [False, True])
def test_linear_qkv_rope_store(ops, heads, kv_heads, head_dim, rotary, hidden, q_lens, starts, deferred):
    """The q/k/v product fused with bias, rotation and the cache store, for small batches (one kernel adds the
    product's partial sums, rotates and stores) and larger ones (separate kernels), with rows that still lack
    their norm factor and with complete ones, at two head sizes, with a full, a partial and no rotation."""
    from aegean_tge_b200.parts.rope import rotary_tables
    page_size = 16
    positions, seq_of_token, _, _ = batch_index(q_lens, starts, DEV)
    T = sum(q_lens)
    width = (heads + 2 * kv_heads) * head_dim
    gen = torch.Generator().manual_seed(heads * 10 + head_dim + T)
    x = torch.randn(T, hidden, generator=gen).to(torch.bfloat16)
    w = (torch.randn(width, hidden, generator=gen) * 0.1).to(torch.bfloat16)
    bias = torch.randn(width, generator=gen)
    lengths = [s + n for s, n in zip(starts, q_lens)]
    cos = sin = None
    if rotary:
        cos, sin = rotary_tables(12345.0, rotary, 96)
    taken = x
    normed = x.double()
    if deferred and T <= 128:
        # rows = stream * gain in bfloat16 plus the sums of squares of the stream in slices: what linear_add_norm hands on
        stream = torch.randn(T, hidden, generator=gen) * 2.0
        gain = 1.0 + 0.2 * torch.randn(hidden, generator=gen)
        rows = (stream * gain).to(torch.bfloat16)
        slices = -(-hidden // 96)
        sums = torch.stack([(stream[:, i * 96:(i + 1) * 96].double() ** 2).sum(1) for i in range(slices)]).float()
        taken = ops.DeferredRows(rows.to(DEV), sums.to(DEV).contiguous(), hidden, 1e-5)
        normed = rows.double() / torch.sqrt((stream.double() ** 2).mean(1, keepdim=True) + 1e-5)
    qkv_ref = ops_plain.linear(normed, w, bias)
    pos = positions.cpu().long()
    q = qkv_ref[:, :heads * head_dim].view(T, heads, head_dim)
    k = qkv_ref[:, heads * head_dim:(heads + kv_heads) * head_dim].view(T, kv_heads, head_dim)
    v = qkv_ref[:, (heads + kv_heads) * head_dim:].view(T, kv_heads, head_dim)
    c = cos[pos] if rotary else None
    s = sin[pos] if rotary else None
    q_ref, k_ref = ops_plain.rotate_half(q, c, s, rotary), ops_plain.rotate_half(k, c, s, rotary)
    for _ in range(1):
        k_pages, v_pages, table, _, _ = paged_cache(lengths, kv_heads, head_dim, page_size, torch.bfloat16, DEV, seed=4)
        before_k = k_pages.clone()
        out = ops.linear_qkv_rope_store(taken if not isinstance(taken, torch.Tensor) else taken.to(DEV), w.to(DEV),
                                        bias.to(DEV), None if cos is None else cos.to(DEV),
                                        None if sin is None else sin.to(DEV), rotary, positions, seq_of_token, table,
                                        k_pages, v_pages, heads, kv_heads, head_dim)
        ops.check_status()
        assert rel_error(out[:, :heads * head_dim].reshape(T, heads, head_dim), q_ref) < TOL[torch.bfloat16]
        touched = torch.zeros_like(before_k, dtype=torch.bool)
        for t in range(T):
            page = int(table[int(seq_of_token[t]), int(pos[t]) // page_size])
            slot = int(pos[t]) % page_size
            assert rel_error(k_pages[page, :, slot], k_ref[t]) < TOL[torch.bfloat16]
            assert rel_error(v_pages[page, :, slot], v[t]) < TOL[torch.bfloat16]
            touched[page, :, slot] = True
        assert torch.equal(k_pages[~touched], before_k[~touched]), "a slot outside the step's positions was written"


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------
def _attention_case(ops, dtype, heads, kv_heads, head_dim, q_lens, starts, window=0, split=0, force_simt=False,
                    page_size=16, spike=None, decode_prefix=0):
    lengths = [s + n for s, n in zip(starts, q_lens)]
    k_pages, v_pages, table, k_list, v_list = paged_cache(lengths, kv_heads, head_dim, page_size, dtype, DEV, seed=9)
    positions, seq_of_token, q_start, start_pos = batch_index(q_lens, starts, DEV)
    T = sum(q_lens)
    gen = torch.Generator().manual_seed(17)
    stride = heads * head_dim + 24          # rows wider than the queries, as inside a fused qkv buffer
    buf = torch.randn(T, stride, generator=gen).to(dtype)
    if spike is not None:
        # make one (far) key of request 0 dominate the first query head of its last row
        seq, key_pos = spike
        row = sum(q_lens[:seq + 1]) - 1
        direction = k_list[seq][key_pos, 0].float()
        buf[row, :head_dim] = (direction / direction.norm() * 60.0).to(dtype)
    scale = 1.0 / math.sqrt(head_dim)
    dq = buf.to(DEV)
    out = ops.attention(dq[:, :heads * head_dim], k_pages, v_pages, table, q_start, start_pos, positions,
                        seq_of_token, len(q_lens), max(q_lens), max(lengths), heads, kv_heads, head_dim, scale,
                        window=window, split_tokens=split, force_simt=force_simt, decode_prefix=decode_prefix)
    ops.check_status()
    q = buf[:, :heads * head_dim].view(T, heads, head_dim)
    refs = []
    for s, (n, start) in enumerate(zip(q_lens, starts)):
        begin = sum(q_lens[:s])
        refs.append(ops_plain.attention_rows(q[begin:begin + n], k_list[s], v_list[s], range(start, start + n),
                                             scale, window))
    ref = torch.cat(refs).reshape(T, heads * head_dim)
    return rel_error(out, ref), out, ref


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim", [(6, 2, 48), (3, 1, 32), (4, 4, 16), (7, 1, 128), (2, 2, 100)])
def test_attention_simt(ops, dtype, heads, kv_heads, head_dim):
    err, _, _ = _attention_case(ops, dtype, heads, kv_heads, head_dim, [5, 1, 37, 2], [30, 150, 0, 63],
                                force_simt=True)
    assert err < TOL[dtype]


def test_leading_single_tokens_deep_in_long_contexts_get_splits_of_their_own(ops):
    """A mixed step: nine single tokens at contexts of about 4,000 beside a prompt of 300 tokens.  The prompt's
    keys are not cut; the single tokens, a decode batch of their own, have theirs cut (the choice is automatic
    here), and one far key dominates a row so that a split lost in the merge would show."""
    starts = [4000 + 37 * i for i in range(9)] + [0]
    err, _, _ = _attention_case(ops, torch.bfloat16, 14, 2, 128, [1] * 9 + [300], starts, decode_prefix=9, spike=(0, 123))
    assert err < TOL[torch.bfloat16]
    assert ops.choose_attention_split(9, 9, 1, 4400, 14, 2, bound=4400) > 0          # the single tokens' keys are cut
    starts = [4000 + 37 * i for i in range(9)] + [2900]                                # ... also beside a long portion
    err, _, _ = _attention_case(ops, torch.bfloat16, 14, 2, 128, [1] * 9 + [1500], starts, decode_prefix=9, spike=(0, 123))
    assert err < TOL[torch.bfloat16]
    assert ops.choose_attention_split(1509, 10, 1500, 4400, 14, 2, bound=4400) == 0  # whose keys are not cut


@pytest.mark.parametrize("split,window", [(256, 0), (128, 0), (64, 0), (64, 700)])
def test_attention_merges_many_splits(ops, split, window):
    """Single tokens deep in a context, their keys cut into 14, 28 and 55 splits: the merging kernel holds up to 16
    or 48 split states in registers and walks more than that in a loop; with a window most splits hold no
    visible key.  One far key is made to dominate, so a split dropped or counted twice would show."""
    err, _, _ = _attention_case(ops, torch.bfloat16, 14, 2, 128, [1, 1, 1], [3499, 1200, 65], window=window, split=split,
                                spike=(0, 3000 if window else 17))
    assert err < TOL[torch.bfloat16]


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(7, 1, 128), (28, 4, 64), (6, 2, 48), (40, 2, 16)])
@pytest.mark.parametrize("page_size,split,window", [(16, 0, 0), (64, 128, 0), (4, 64, 0), (16, 0, 40), (32, 64, 100)])
def test_attention_routes_leading_single_tokens_to_the_decode_kernel(ops, heads, kv_heads, head_dim, page_size, split,
                                                                     window):
    """A step whose first ten sequences bring one token each and whose last two bring portions: told so, the
    tensor-core path serves the ten with its decode kernel and the rest with its prefill kernel (with and without
    a cut of the keys, whose partial results share one scratch buffer); untold, one kernel serves all.  Both are
    right, and they agree to rounding.  One single token sits at position 0, one far into its sequence; with a
    window some splits hold no visible key."""
    q_lens = [1] * 10 + [70, 3]
    starts = [0, 199, 64, 5, 130, 17, 63, 64, 255, 1] + [200, 15]
    routed, out_routed, _ = _attention_case(ops, torch.bfloat16, heads, kv_heads, head_dim, q_lens, starts, split=split,
                                            page_size=page_size, decode_prefix=10, window=window)
    plain_way, out_plain, _ = _attention_case(ops, torch.bfloat16, heads, kv_heads, head_dim, q_lens, starts, split=split,
                                              page_size=page_size, window=window)
    assert routed < TOL[torch.bfloat16] and plain_way < TOL[torch.bfloat16]
    assert rel_error(out_routed, out_plain.float()) < TOL[torch.bfloat16]


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(6, 2, 48), (3, 1, 32), (4, 4, 16), (7, 1, 128), (28, 4, 64),
                                                     (5, 5, 80), (40, 2, 16), (4, 2, 256), (6, 2, 192)])
@pytest.mark.parametrize("q_lens,starts", [([5, 1, 37, 2], [30, 150, 0, 63]), ([1, 1, 1], [0, 199, 64]),
                                           ([130], [0]), ([70, 3], [200, 15])])
def test_attention_mma(ops, heads, kv_heads, head_dim, q_lens, starts):
    err, _, _ = _attention_case(ops, torch.bfloat16, heads, kv_heads, head_dim, q_lens, starts)
    assert err < TOL[torch.bfloat16]


@pytest.mark.parametrize("split", [64, 128, 192])
@pytest.mark.parametrize("q_lens,starts", [([1, 1, 1, 1], [700, 3, 255, 256]), ([40, 1], [300, 129])])
def test_attention_mma_split_keys(ops, split, q_lens, starts):
    err, _, _ = _attention_case(ops, torch.bfloat16, 7, 1, 128, q_lens, starts, split=split)
    assert err < TOL[torch.bfloat16]
    err, _, _ = _attention_case(ops, torch.bfloat16, 6, 2, 48, q_lens, starts, split=split)
    assert err < TOL[torch.bfloat16]


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(28, 4, 128), (10, 2, 64), (16, 1, 128)])
@pytest.mark.parametrize("split,window", [(128, 0), (512, 0), (256, 300), (64, 0), (192, 77)])
def test_attention_decode_splits(ops, heads, kv_heads, head_dim, split, window):
    """Single tokens with two to sixteen key splits, some of them without keys for the short requests."""
    err, _, _ = _attention_case(ops, torch.bfloat16, heads, kv_heads, head_dim, [1, 1, 1, 1, 1], [1000, 0, 511, 512, 130],
                                window=window, split=split)
    assert err < TOL[torch.bfloat16]


@pytest.mark.parametrize("dtype,simt", [(torch.float32, True), (torch.bfloat16, True), (torch.bfloat16, False)])
def test_attention_reads_a_far_key(ops, dtype, simt):
    """One key hundreds of positions back carries almost all the weight: the output must be its value."""
    err, out, ref = _attention_case(ops, dtype, 4, 2, 64, [1, 3], [600, 20], force_simt=simt, spike=(0, 7))
    assert err < TOL[dtype]


@pytest.mark.parametrize("dtype,simt", [(torch.float32, True), (torch.bfloat16, False)])
@pytest.mark.parametrize("window", [1, 16, 40, 65])
def test_attention_window_edge(ops, dtype, simt, window):
    """With a window the key just outside it must not count, however strong; the one just inside must."""
    for key_offset in (window, window - 1):           # just outside / just inside (distance from the query)
        start = 300
        if key_offset > start:
            continue
        err, out, ref = _attention_case(ops, dtype, 4, 2, 64, [1, 5], [start, 100], window=window, force_simt=simt,
                                        spike=(0, start - key_offset))
        assert err < TOL[dtype]
    err, _, _ = _attention_case(ops, dtype, 4, 2, 64, [33, 2], [60, 10], window=window, force_simt=simt, split=64 if not simt else 0)
    assert err < TOL[dtype]


# ---------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------
def test_sample_greedy_takes_the_first_maximum(ops):
    logits = torch.zeros(3, 1000)
    logits[0, 17] = 5.0
    logits[0, 800] = 5.0                         # a tie: the lower index wins (sampling.cpp:198-207)
    logits[1, 999] = 1.0
    logits[2, :] = -3.0                          # all equal: index 0
    ids = ops.sample(logits.to(DEV), torch.zeros(3, device=DEV), torch.zeros(3, device=DEV))
    assert ids.cpu().tolist() == [17, 999, 0]


@pytest.mark.parametrize("vocab", [331, 4097, 152064])
def test_sample_temperature_lands_where_the_draw_points(ops, vocab):
    """The chosen index is the one whose slice of the exact (float64) cumulative distribution holds the
    draw u.  Float32 sums over n terms are exact to about n * 2^-24 of the total, so the draw may sit
    that far outside the chosen slice, no further; on a small vocabulary the kernel must also agree
    with the sequential float32 walk of the reference."""
    from plain.qwen2_plain import sample_plain
    import numpy as np
    gen = torch.Generator().manual_seed(vocab)
    rows = 6
    logits = torch.randn(rows, vocab, generator=gen) * 2.0
    temps = [0.8, 1.0, 0.3, 2.0, 0.8, 0.05]
    uniforms = [0.37, 0.9991, 0.0004, 0.5, 0.73, 0.11]
    ids = ops.sample(logits.to(DEV), torch.tensor(temps, device=DEV), torch.tensor(uniforms, device=DEV)).cpu().tolist()
    slack = vocab * 2.0 ** -24

    class Fixed:
        def __init__(self, u): self.u = u
        def next(self): return np.float32(self.u)
    for r in range(rows):
        z = logits[r].double()
        e = torch.exp((z - z.max()) / temps[r])
        cdf = torch.cumsum(e, 0) / e.sum()
        lower = float(cdf[ids[r] - 1]) if ids[r] > 0 else 0.0
        assert lower - slack <= uniforms[r] <= float(cdf[ids[r]]) + slack, (r, ids[r], lower, float(cdf[ids[r]]))
        if vocab <= 4097:
            assert ids[r] == sample_plain(logits[r].numpy(), temps[r], Fixed(uniforms[r]))


def test_sample_histogram_follows_the_distribution(ops):
    """Many draws from a small distribution: observed frequencies within a chi-square bound."""
    from aegean_tge_b200.sampling import XorShift32
    probs = torch.tensor([0.5, 0.25, 0.125, 0.0625, 0.0625])
    logits = torch.log(probs)[None, :].repeat(4000, 1)
    rng = XorShift32(123)
    uniforms = torch.tensor([rng.next_uniform() for _ in range(4000)])
    ids = ops.sample(logits.to(DEV), torch.ones(4000, device=DEV), uniforms.to(DEV)).cpu()
    counts = torch.bincount(ids.long(), minlength=5).double()
    expected = probs.double() * 4000
    chi2 = float(((counts - expected) ** 2 / expected).sum())
    assert chi2 < 20.5          # 4 degrees of freedom, p ~ 4e-4


def test_a_bounded_wait_gives_up_and_leaves_the_device_usable():
    """The product kernels wait on barriers with a time limit; when it runs out they set a status bit and
    unwind instead of hanging.  A one-thread kernel makes that wait run out on purpose (a barrier nothing
    arrives at, a limit of 1 ms): the launch returns, the status word says so once, and a product right
    afterwards is exact."""
    from aegean_tge_b200 import ops
    ops.check_status()
    arrived, took = ops.wait_gives_up(1_000_000)
    torch.cuda.synchronize()
    assert not arrived and 1_000_000 <= took < 50_000_000, (arrived, took)
    with pytest.raises(ops.DeviceStatusError, match="wait gave up"):
        ops.check_status()
    ops.check_status()                                  # reading it cleared it
    with pytest.raises(ops.KernelError):
        ops.wait_gives_up(10**9)                        # long limits are refused outright
    x = torch.randint(-3, 4, (24, 256), device="cuda").to(torch.bfloat16)
    w = torch.randint(-3, 4, (384, 256), device="cuda").to(torch.bfloat16)
    out = ops.linear(x, w, None, ops.GEMM_STORE_F32)
    assert torch.equal(out, x.float() @ w.float().T)    # small integers: exact in bfloat16 products and float32 sums
    ops.check_status()
