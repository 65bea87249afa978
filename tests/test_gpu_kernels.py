"""Each kernel alone against a plain PyTorch fp32/fp64 restatement of the same operation, at sizes
other than the engine's test models."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def K():
    from burn_lm_b200 import kernels
    return kernels


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("table_dtype", DTYPES)
def test_embed(table_dtype):
    g = torch.Generator(device="cuda").manual_seed(0)
    table = torch.randn(301, 72, device="cuda", generator=g).to(table_dtype)
    tokens = torch.randint(0, 301, (17,), device="cuda", generator=g, dtype=torch.int32)
    out = torch.empty(17, 72, device="cuda")
    K().embed(tokens, table, out)
    torch.testing.assert_close(out, table[tokens.long()].float(), rtol=0, atol=0)


@pytest.mark.parametrize("gdt", DTYPES)
@pytest.mark.parametrize("n,width", [(1, 64), (7, 2048), (16, 1000)])
def test_embed_hands_the_first_norm_over(gdt, n, width):
    """With `hand_over` the embedding leaves what the products that write the stream leave: the stream times gamma in
    bfloat16 and the rows' sums of squares (one part), beside the same fp32 rows as without it."""
    k = K()
    g = torch.Generator(device="cuda").manual_seed(n + width)
    table = torch.randn(300, width, device="cuda", generator=g).to(torch.bfloat16)
    tokens = torch.randint(0, 300, (n,), device="cuda", generator=g, dtype=torch.int32)
    gamma = (1 + 0.1 * torch.randn(width, device="cuda", generator=g)).to(gdt)
    plain = torch.empty(n, width, device="cuda")
    k.embed(tokens, table, plain)
    out = torch.empty(n, width, device="cuda")
    scaled = torch.full((n, width), float("nan"), device="cuda", dtype=torch.bfloat16)
    squares = torch.full((1, 16), float("nan"), device="cuda")
    k.embed(tokens, table, out, hand_over=(gamma, scaled, squares))
    assert torch.equal(out, plain) and torch.equal(out, table[tokens.long()].float())
    want = out.double() * gamma.double()
    assert (scaled.double() - want).abs().max().item() <= 2 ** -8 * want.abs().max().item()
    ssq = (out.double() ** 2).sum(-1)
    assert (squares[0, :n].double() - ssq).abs().max().item() < 1e-5 * ssq.max().item()
    with pytest.raises(k.KernelError):
        k.embed(torch.zeros(17, dtype=torch.int32, device="cuda"), table, torch.empty(17, width, device="cuda"),
                hand_over=(gamma, torch.empty(17, width, device="cuda", dtype=torch.bfloat16), squares))


@pytest.mark.parametrize("act", DTYPES)
@pytest.mark.parametrize("gdt", DTYPES)
@pytest.mark.parametrize("width", [72, 1000, 4100])
def test_add_rmsnorm(act, gdt, width):
    g = torch.Generator(device="cuda").manual_seed(1)
    n = 13
    resid = torch.randn(n, width, device="cuda", generator=g)
    delta = torch.randn(n, width, device="cuda", generator=g).to(act)
    gamma = (1 + 0.1 * torch.randn(width, device="cuda", generator=g)).to(gdt)
    eps = 3e-6
    h = resid.double() + delta.double()
    want = h / torch.sqrt((h * h).mean(-1, keepdim=True) + eps) * gamma.double()
    r = resid.clone()
    out = torch.empty(n, width, device="cuda", dtype=act)
    K().add_rmsnorm(r, delta, gamma, eps, out)
    torch.testing.assert_close(r.double(), h, rtol=1e-6, atol=1e-6)       # the sum is stored in fp32
    torch.testing.assert_close(out.double(), want, **tol(act))
    # rows mode leaves the stream alone; a missing delta adds nothing
    rows = torch.tensor([5, 0, 12], device="cuda", dtype=torch.int32)
    r2 = resid.clone()
    out2 = torch.empty(3, width, device="cuda", dtype=act)
    K().add_rmsnorm(r2, delta, gamma, eps, out2, rows)
    torch.testing.assert_close(r2, resid, rtol=0, atol=0)
    torch.testing.assert_close(out2.double(), want[rows.long()], **tol(act))
    out3 = torch.empty(n, width, device="cuda", dtype=act)
    K().add_rmsnorm(r2, None, gamma, eps, out3)
    h0 = resid.double()
    torch.testing.assert_close(out3.double(), h0 / torch.sqrt((h0 * h0).mean(-1, keepdim=True) + eps) * gamma.double(), **tol(act))


def rope_reference(x, pos, inv_freq, rot, interleaved):
    """x [N, heads, hd] float64."""
    ang = pos.double()[:, None] * inv_freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:rot:2], x[..., 1:rot:2]
        out[..., 0:rot:2] = a * c - b * s
        out[..., 1:rot:2] = a * s + b * c
    else:
        a, b = x[..., : rot // 2], x[..., rot // 2: rot]
        out[..., : rot // 2] = a * c - b * s
        out[..., rot // 2: rot] = a * s + b * c
    return out


def paged_setup(lens_before, lens_new, n_kv, hd, dtype, seed, n_pages=None, shuffle=True):
    """Block tables with shuffled pages and a pool full of NaN, as a reused cache would be."""
    k = K()
    g = torch.Generator().manual_seed(seed)
    n_seqs = len(lens_new)
    total = [a + b for a, b in zip(lens_before, lens_new)]
    need = [(t + k.PAGE - 1) // k.PAGE for t in total]
    n_pages = n_pages or sum(need) + 3
    perm = torch.randperm(n_pages, generator=g).tolist() if shuffle else list(range(n_pages))
    max_pages = max(need) + 1
    slots = torch.randperm(n_seqs + 2, generator=g)[:n_seqs].tolist()
    table = torch.zeros(n_seqs + 2, max_pages, dtype=torch.int32)
    it = iter(perm)
    for s in range(n_seqs):
        for p in range(need[s]):
            table[slots[s], p] = next(it)
    pool = torch.full((n_pages, 2, n_kv, k.PAGE, hd), float("nan"), dtype=dtype, device="cuda")
    cu = [0]
    for n in lens_new:
        cu.append(cu[-1] + n)
    token_seq = [s for s, n in enumerate(lens_new) for _ in range(n)]
    token_pos = [lens_before[s] + t for s, n in enumerate(lens_new) for t in range(n)]
    dev = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    return dict(table=table.cuda(), pool=pool, cu=dev(cu), token_seq=dev(token_seq), token_pos=dev(token_pos),
                slots=dev(slots), starts=dev(lens_before), host_table=table, host_slots=slots, total=total)


def write_history(setup, k_hist, v_hist):
    """Put per-sequence history [len, n_kv, hd] into the pool through the block table."""
    P = K().PAGE
    pool = setup["pool"]
    for s, (kh, vh) in enumerate(zip(k_hist, v_hist)):
        pos = torch.arange(kh.shape[0])
        pages = setup["host_table"][setup["host_slots"][s]][pos // P].long().to(pool.device)
        offs = (pos % P).to(pool.device)
        pool[pages, 0, :, offs] = kh.to(pool.dtype)        # [len, n_kv, hd] each
        pool[pages, 1, :, offs] = vh.to(pool.dtype)


def read_history(setup, s, length):
    P = K().PAGE
    ks, vs = [], []
    for pos in range(length):
        page = int(setup["host_table"][setup["host_slots"][s], pos // P])
        ks.append(setup["pool"][page, 0, :, pos % P])
        vs.append(setup["pool"][page, 1, :, pos % P])
    return torch.stack(ks), torch.stack(vs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("hd,rot", [(48, 48), (32, 16), (64, 0)])
def test_rope_append(dtype, interleaved, hd, rot):
    k = K()
    H, KV = 5, 3
    lens_before, lens_new = [0, 70, 63, 129], [9, 1, 3, 66]
    st = paged_setup(lens_before, lens_new, KV, hd, dtype, seed=2)
    n = sum(lens_new)
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(n, (H + 2 * KV) * hd, device="cuda", generator=g).to(dtype)
    inv_freq = None
    if rot:
        inv_freq = torch.tensor([1e4 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64, device="cuda")
    before = qkv.clone()
    k.rope_append(qkv, st["token_seq"], st["token_pos"], st["slots"], st["table"], inv_freq, rot, interleaved,
                  st["pool"], H, KV, hd)
    x = before.double().view(n, H + 2 * KV, hd)
    want_q = x[:, :H]
    want_k = x[:, H:H + KV]
    if rot:
        want_q = rope_reference(want_q, st["token_pos"], inv_freq, rot, interleaved)
        want_k = rope_reference(want_k, st["token_pos"], inv_freq, rot, interleaved)
    t = tol(dtype)
    torch.testing.assert_close(qkv.double().view(n, H + 2 * KV, hd)[:, :H], want_q, **t)
    # k and v sit at their positions in the pages
    row = 0
    for s, new in enumerate(lens_new):
        kh, vh = read_history(st, s, st["total"][s])
        torch.testing.assert_close(kh[lens_before[s]:].double(), want_k[row:row + new], **t)
        torch.testing.assert_close(vh[lens_before[s]:].double(), x[row:row + new, H + KV:], rtol=0, atol=0)
        assert torch.isnan(kh[: lens_before[s]].float()).all()      # nothing else was touched
        row += new


def attention_reference(q, k_all, v_all, start, scale, window):
    """q [T, H, hd], k_all/v_all [S, KV, hd] float64; token t at position start + t."""
    T, H, hd = q.shape
    S, KV, _ = k_all.shape
    G = H // KV
    out = torch.empty_like(q)
    for h in range(H):
        s = (q[:, h] @ k_all[:, h // G].T) * scale
        i = torch.arange(T, device=q.device)[:, None] + start
        j = torch.arange(S, device=q.device)[None, :]
        hidden = j > i
        if window:
            hidden = hidden | (j <= i - window)
        s = s.masked_fill(hidden, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v_all[:, h // G]
    return out


def run_attention_case(dtype, H, KV, hd, lens_before, lens_new, window, n_splits, seed, max_kv_len=0):
    k = K()
    st = paged_setup(lens_before, lens_new, KV, hd, dtype, seed=seed)
    g = torch.Generator(device="cuda").manual_seed(seed + 100)
    n = sum(lens_new)
    q_stride = (H + 2 * KV) * hd
    qkv = torch.randn(n, q_stride, device="cuda", generator=g).to(dtype)
    k_hist = [torch.randn(t, KV, hd, device="cuda", generator=g).to(dtype) for t in st["total"]]
    v_hist = [torch.randn(t, KV, hd, device="cuda", generator=g).to(dtype) for t in st["total"]]
    write_history(st, k_hist, v_hist)
    out = torch.empty(n, H * hd, device="cuda", dtype=dtype)
    scale = 1.0 / math.sqrt(hd)
    scratch = None
    if n_splits > 1:
        scratch = torch.empty(k.attention_scratch_floats(n, H, hd, n_splits), device="cuda")
    k.attention(qkv, q_stride, st["pool"], st["table"], st["cu"], st["slots"], st["starts"], out, n, len(lens_new),
                max(lens_new), H, KV, hd, scale, window=window, n_splits=n_splits, scratch=scratch, max_kv_len=max_kv_len)
    k.check_status("cuda")
    if dtype == torch.bfloat16 and (max(lens_new) == 1 or max(lens_new) >= 16):
        # whichever kernel took the step, the general one must say the same (up to bf16 rounding of the output)
        out_general = torch.empty_like(out)
        k.attention(qkv, q_stride, st["pool"], st["table"], st["cu"], st["slots"], st["starts"], out_general, n, len(lens_new),
                    max(lens_new), H, KV, hd, scale, window=window, n_splits=n_splits, scratch=scratch, general_only=True)
        torch.testing.assert_close(out.float(), out_general.float(), rtol=2e-2, atol=1e-2)
    row = 0
    for s, new in enumerate(lens_new):
        q = qkv[row:row + new].double().view(new, -1, hd)[:, :H]
        want = attention_reference(q, k_hist[s].double(), v_hist[s].double(), lens_before[s], scale, window)
        got = out[row:row + new].double().view(new, H, hd)
        assert not torch.isnan(got).any()
        torch.testing.assert_close(got, want, **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)))
        row += new


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,hd", [(4, 2, 16), (6, 1, 32), (5, 5, 48), (8, 2, 128), (3, 1, 256), (40, 1, 64)])
def test_attention_prompts(dtype, H, KV, hd):
    run_attention_case(dtype, H, KV, hd, [0, 0, 0, 0], [1, 7, 64, 131], 0, 1, seed=5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,hd", [(4, 2, 16), (6, 1, 32), (32, 8, 64), (7, 7, 80)])
@pytest.mark.parametrize("n_splits", [1, 3, 8])
def test_attention_single_tokens(dtype, H, KV, hd, n_splits):
    run_attention_case(dtype, H, KV, hd, [0, 63, 64, 300, 129], [1, 1, 1, 1, 1], 0, n_splits, seed=6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_continued_prompts_and_window(dtype):
    run_attention_case(dtype, 6, 2, 32, [10, 100, 64], [5, 40, 70], 0, 1, seed=7)
    run_attention_case(dtype, 6, 2, 32, [10, 100, 64], [5, 40, 70], 37, 1, seed=8)
    run_attention_case(dtype, 6, 2, 32, [200, 70, 5], [1, 1, 1], 65, 4, seed=9)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key(dtype):
    """One key among hundreds is made to match the query: the output must be that key's value."""
    k = K()
    H, KV, hd, S = 4, 2, 64, 700
    for target in (0, 63, 64, 377, 699):
        for n_splits in (1, 5):
            st = paged_setup([S - 1], [1], KV, hd, dtype, seed=target)
            g = torch.Generator(device="cuda").manual_seed(11)
            kh = (0.01 * torch.randn(S, KV, hd, device="cuda", generator=g)).to(dtype)
            vh = torch.randn(S, KV, hd, device="cuda", generator=g).to(dtype)
            q = torch.zeros(1, (H + 2 * KV) * hd, device="cuda", dtype=dtype)
            q[0, : H * hd] = 1.0
            kh[target] = 4.0
            write_history(st, [kh], [vh])
            out = torch.empty(1, H * hd, device="cuda", dtype=dtype)
            scratch = torch.empty(max(1, k.attention_scratch_floats(1, H, hd, n_splits)), device="cuda")
            k.attention(q, q.shape[1], st["pool"], st["table"], st["cu"], st["slots"], st["starts"], out, 1, 1, 1,
                        H, KV, hd, 1.0, n_splits=n_splits, scratch=scratch)
            want = vh[target].float().repeat_interleave(H // KV, dim=0).reshape(-1)
            torch.testing.assert_close(out[0].float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    g = torch.Generator(device="cuda").manual_seed(12)
    gu = torch.randn(11, 2 * 200, device="cuda", generator=g).to(dtype)
    out = torch.empty(11, 200, device="cuda", dtype=dtype)
    K().swiglu(gu, out)
    a, b = gu.double()[:, :200], gu.double()[:, 200:]
    torch.testing.assert_close(out.double(), a / (1 + torch.exp(-a)) * b, **tol(dtype))


@pytest.mark.parametrize("n,m,k_", [(1, 7, 5), (65, 130, 33), (200, 300, 1000)])
def test_gemm_f32(n, m, k_):
    g = torch.Generator(device="cuda").manual_seed(13)
    x = torch.randn(n, k_, device="cuda", generator=g)
    w = torch.randn(m, k_, device="cuda", generator=g)
    y = K().gemm_f32(x, w)
    torch.testing.assert_close(y.double(), x.double() @ w.double().T, rtol=1e-5, atol=1e-4)
    # a row's result does not depend on the other rows of the batch
    y1 = K().gemm_f32(x[:1].contiguous(), w)
    assert torch.equal(y1[0], y[0])


def test_convert():
    x = torch.randn(1000, device="cuda")
    b = torch.empty(1000, device="cuda", dtype=torch.bfloat16)
    K().convert(x, b)
    assert torch.equal(b, x.to(torch.bfloat16))
    f = torch.empty(1000, device="cuda")
    K().convert(b, f)
    assert torch.equal(f, b.float())


def test_argmax_lowest_index_wins():
    g = torch.Generator(device="cuda").manual_seed(14)
    logits = torch.randn(5, 5003, device="cuda", generator=g)
    logits[1, 4000] = logits[1, 17] = 50.0
    logits[2, 5002] = 60.0
    out = torch.empty(5, device="cuda", dtype=torch.int32)
    K().argmax(logits, out)
    want = logits.argmax(-1)
    want[1] = 17
    assert out.tolist() == want.tolist()


def test_refusals():
    k = K()
    with pytest.raises(k.KernelError):
        k.embed(torch.zeros(3, dtype=torch.int32), torch.zeros(4, 4), torch.zeros(3, 4))   # CPU tensors
    q = torch.zeros(1, 3 * 24, device="cuda")
    pool = torch.zeros(2, 2, 1, k.PAGE, 24, device="cuda")
    z = torch.zeros(2, dtype=torch.int32, device="cuda")
    with pytest.raises(k.KernelError, match="multiple of 16"):
        k.attention(q, 72, pool, z.view(1, 2), z, z, z, torch.zeros(1, 24, device="cuda"), 1, 1, 1, 1, 1, 24, 1.0)


def gemv_reference(w, x):
    return x.double() @ w.double().T


@pytest.mark.parametrize("n", [1, 3, 8, 9, 16])
# (18944, 2048): eight tiles for every block, all warps busy; (40016, 512): several rounds, the last one partial
@pytest.mark.parametrize("m,k", [(40, 64), (200, 192), (3072, 2048), (1000, 8192), (77, 4160), (2500, 512), (18944, 2048), (40016, 512),
                                 (4096, 14336)])
def test_gemv_store(n, m, k):
    g = torch.Generator(device="cuda").manual_seed(n * 1000 + m)
    w = (torch.randn(m, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    x = torch.randn(n, k, device="cuda", generator=g).to(torch.bfloat16)
    if not K().gemv_supported(n, m, k, plain_tokens=True):
        assert n > 8 and k >= 8192          # only: too many tokens of too wide rows for shared memory
        pytest.skip("the tokens do not fit shared memory; the library product takes this shape")
    want = gemv_reference(w, x)
    scale = want.abs().max().item()
    out32 = torch.empty(n, m, device="cuda")
    K().gemv(w, n, x=x, out=out32)
    assert (out32.double() - want).abs().max().item() < 2e-5 * scale + 1e-6     # fp32 accumulation of exact products
    out16 = torch.empty(n, m, device="cuda", dtype=torch.bfloat16)
    K().gemv(w, n, x=x, out=out16)
    assert (out16.double() - want).abs().max().item() < 5e-3 * scale
    # a token's result does not depend on the other tokens of the batch
    one = torch.empty(1, m, device="cuda")
    K().gemv(w, 1, x=x[:1].contiguous(), out=one)
    assert torch.equal(one[0], out32[0])
    K().check_status("cuda")


@pytest.mark.parametrize("n", [1, 8, 16])
@pytest.mark.parametrize("gdt", DTYPES)
def test_gemv_norm_prologue_swiglu_and_stream_add(n, gdt):
    g = torch.Generator(device="cuda").manual_seed(n)
    k, inner, m = 192, 576, 192
    resid = torch.randn(n + 3, k, device="cuda", generator=g)
    gamma = (1 + 0.1 * torch.randn(k, device="cuda", generator=g)).to(gdt)
    rows = torch.randperm(n + 3, device="cuda", generator=g)[:n].to(torch.int32)
    eps = 1e-5
    h = resid.double()[rows.long()]
    xn = (h / torch.sqrt((h * h).mean(-1, keepdim=True) + eps) * gamma.double()).to(torch.bfloat16)   # rounded as the kernel rounds
    wgu = (torch.randn(2 * inner, k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)        # [gate; up]
    tiled = torch.stack([wgu[:inner].view(inner // 8, 8, k), wgu[inner:].view(inner // 8, 8, k)], dim=1).reshape(2 * inner, k).contiguous()
    act = torch.empty(n, inner, device="cuda", dtype=torch.bfloat16)
    K().gemv(tiled, n, stream_rows=resid, gamma=gamma, eps=eps, rows=rows, out=act, swiglu=True)
    gu = gemv_reference(wgu, xn)
    want = gu[:, :inner] / (1 + torch.exp(-gu[:, :inner])) * gu[:, inner:]
    # the element-wise kernel reads the same tiled layout
    act2 = torch.empty(n, inner, device="cuda", dtype=torch.bfloat16)
    K().swiglu(gemv_reference(tiled, xn).to(torch.bfloat16), act2, tile=8)
    assert (act2.double() - want).abs().max().item() < 2e-2 * want.abs().max().item()
    assert (act.double() - want).abs().max().item() < 1e-2 * want.abs().max().item()
    # without rows, and adding into the stream
    wd = (torch.randn(m, inner, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    stream = torch.randn(n, m, device="cuda", generator=g)
    before = stream.clone()
    K().gemv(wd, n, x=act, add_into=stream)
    want2 = before.double() + gemv_reference(wd, act)
    assert (stream.double() - want2).abs().max().item() < 2e-5 * want2.abs().max().item()
    out = torch.empty(n, m, device="cuda")
    K().gemv(wd[:, :k].contiguous(), n, stream_rows=resid[:n].contiguous(), gamma=gamma, eps=eps, out=out)
    h2 = resid.double()[:n]
    xn2 = (h2 / torch.sqrt((h2 * h2).mean(-1, keepdim=True) + eps) * gamma.double()).to(torch.bfloat16)
    want3 = gemv_reference(wd[:, :k], xn2)
    assert (out.double() - want3).abs().max().item() < 1e-3 * want3.abs().max().item()


@pytest.mark.parametrize("n", [1, 5, 8, 16])
@pytest.mark.parametrize("gdt", DTYPES)
@pytest.mark.parametrize("width,inner", [(192, 320), (2048, 512), (200 * 16 + 8, 64)])
def test_gemv_hands_the_next_norm_over(n, gdt, width, inner):
    """The product that adds into the stream also leaves bfloat16(stream * gamma) and the rows' sums of
    squares by tiles; the product after it takes those instead of normalising the stream itself."""
    g = torch.Generator(device="cuda").manual_seed(n + width)
    act = torch.randn(n, inner, device="cuda", generator=g).to(torch.bfloat16)
    wd = (torch.randn(width, inner, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(width, device="cuda", generator=g)).to(gdt)
    stream = torch.randn(n, width, device="cuda", generator=g) * 3
    stream[n // 2, 7] = 40.0           # one lane that dominates its row's sum of squares
    before = stream.clone()
    scaled = torch.full((n, width), float("nan"), device="cuda", dtype=torch.bfloat16)
    squares = torch.full(((width + 15) // 16, 16), float("nan"), device="cuda")
    K().gemv(wd, n, x=act, add_into=stream, hand_over=(gamma, scaled, squares))
    new = before.double() + gemv_reference(wd, act)
    assert (stream.double() - new).abs().max().item() < 2e-5 * new.abs().max().item()
    want_scaled = stream.double() * gamma.double()
    assert (scaled.double() - want_scaled).abs().max().item() <= 2 ** -8 * want_scaled.abs().max().item()
    assert (squares[:, :n].double().sum(0) - (stream.double() ** 2).sum(-1)).abs().max().item() < 1e-5 * (stream.double() ** 2).sum(-1).max().item()
    # the consumer: gathers rows, divides by the root mean square
    eps = 1e-5
    m = 136
    w2 = (torch.randn(m, width, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    if width % 64:
        return          # the producer takes any width; the consumer's K must be a multiple of 64
    rows = torch.randperm(n, device="cuda", generator=g).to(torch.int32)
    out = torch.empty(n, m, device="cuda")
    K().gemv(w2, n, x=scaled, squares=squares, eps=eps, rows=rows, out=out)
    h = stream.double()[rows.long()]
    want = gemv_reference(w2, scaled[rows.long()]) / torch.sqrt((h * h).mean(-1, keepdim=True) + eps)
    assert (out.double() - want).abs().max().item() < 1e-4 * want.abs().max().item()
    # and it is the norm: against the stream normalised in one piece, up to bfloat16 rounding of the input
    xn = h / torch.sqrt((h * h).mean(-1, keepdim=True) + eps) * gamma.double()
    want_norm = xn @ w2.double().T
    assert (out.double() - want_norm).abs().max().item() < 2e-2 * want_norm.abs().max().item()
    # one token alone gives the same bits as in the batch
    one = torch.empty(1, m, device="cuda")
    K().gemv(w2, 1, x=scaled, squares=squares, eps=eps, rows=rows[:1].contiguous(), out=one)
    assert torch.equal(one[0], out[0])
    K().check_status("cuda")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd", [32, 64, 112])
def test_rope_tiled_pairs(dtype, hd):
    """Pairs dealt out in tiles (eight lanes, then their eight partners) rotate like the pairs
    (i, i + hd / 2) they came from: both kernels, with and without a table."""
    k = K()
    H, KV = 3, 2
    lens_before, lens_new = [0, 70, 5], [9, 1, 66]
    order = torch.tensor(k.tiled_pair_order(hd), device="cuda")
    inv_freq = torch.tensor([1e4 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(hd)
    n = sum(lens_new)
    qkv = torch.randn(n, (H + 2 * KV) * hd, device="cuda", generator=g).to(dtype)
    dealt = qkv.clone().view(n, H + 2 * KV, hd)
    dealt[:, : H + KV] = dealt[:, : H + KV][:, :, order]
    dealt = dealt.reshape(n, -1).contiguous()
    for table_len in (0, 40, 200):          # no table; one that covers some positions; one that covers the step
        a, b = qkv.clone(), dealt.clone()
        sa = paged_setup(lens_before, lens_new, KV, hd, dtype, seed=3)
        sb = paged_setup(lens_before, lens_new, KV, hd, dtype, seed=3)
        table = k.rope_table(inv_freq, table_len) if table_len else None
        mp = max(x + y for x, y in zip(lens_before, lens_new)) - 1
        k.rope_append(a, sa["token_seq"], sa["token_pos"], sa["slots"], sa["table"], inv_freq, hd, k.PAIRS_HALVES, sa["pool"], H, KV, hd,
                      table=table, max_position=mp)
        k.rope_append(b, sb["token_seq"], sb["token_pos"], sb["slots"], sb["table"], inv_freq, hd, k.PAIRS_TILED, sb["pool"], H, KV, hd,
                      table=table, max_position=mp)
        want = a.view(n, H + 2 * KV, hd).clone()
        want[:, : H + KV] = want[:, : H + KV][:, :, order]
        tol = dict(rtol=0, atol=0) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)   # the vector kernel fuses a product
        torch.testing.assert_close(b.view(n, H + 2 * KV, hd)[:, :H].float(), want[:, :H].float(), **tol)
        pa, pb = torch.nan_to_num(sa["pool"].float()), torch.nan_to_num(sb["pool"].float())
        torch.testing.assert_close(pb[:, 0], pa[:, 0][..., order], **tol)
        assert torch.equal(pb[:, 1], pa[:, 1])
        assert torch.equal(torch.isnan(sa["pool"].float()), torch.isnan(sb["pool"].float()))


@pytest.mark.parametrize("n", [1, 7, 16])
@pytest.mark.parametrize("H,KV,hd,width", [(4, 2, 64, 256), (3, 1, 32, 192), (6, 3, 128, 512)])
@pytest.mark.parametrize("write_cache", [True, False])
def test_gemv_rotary_epilogue(n, H, KV, hd, width, write_cache):
    """The skinny product that rotates q and k and appends k and v in its epilogue, against the plain
    product followed by the rotary kernel."""
    k = K()
    g = torch.Generator(device="cuda").manual_seed(n * 7 + hd)
    heads = H + (2 * KV if write_cache else 0)
    w = (torch.randn(heads * hd, width, device="cuda", generator=g) * 0.08).to(torch.bfloat16)
    x = torch.randn(n, width, device="cuda", generator=g).to(torch.bfloat16)
    order = torch.tensor(k.tiled_pair_order(hd), device="cuda")
    dealt = w.clone().view(heads, hd, width)
    dealt[: H + (KV if write_cache else 0)] = dealt[: H + (KV if write_cache else 0)][:, order]
    dealt = dealt.reshape(heads * hd, width).contiguous()
    lens_before = [5 + 37 * i for i in range(n)]                 # one token per sequence, pages 0..n
    inv_freq = torch.tensor([5e5 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64, device="cuda")
    table = k.rope_table(inv_freq, max(lens_before) + 2)
    sa = paged_setup(lens_before, [1] * n, KV, hd, torch.bfloat16, seed=5)
    sb = paged_setup(lens_before, [1] * n, KV, hd, torch.bfloat16, seed=5)
    # the plain way, in the stored order of lanes
    qkv = torch.empty(n, heads * hd, device="cuda", dtype=torch.bfloat16)
    k.gemv(w, n, x=x, out=qkv)
    k.rope_append(qkv, sa["token_seq"], sa["token_pos"], sa["slots"], sa["table"], inv_freq, hd, k.PAIRS_HALVES, sa["pool"], H,
                  KV if write_cache else 0, hd, write_cache=write_cache, table=table, max_position=max(lens_before))
    q_want = qkv[:, : H * hd].reshape(n, H, hd)[:, :, order].float()
    # fused
    q = torch.full((n, H * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
    rope = dict(token_pos=sb["token_pos"], token_seq=sb["token_seq"], slot_of_seq=sb["slots"], block_table=sb["table"], table=table,
                pool=sb["pool"], n_heads=H, n_kv=KV, head_dim=hd, write_cache=write_cache, max_position=max(lens_before))
    k.gemv(dealt, n, x=x, out=q, rope=rope)
    scale = q_want.abs().max().item()
    assert (q.view(n, H, hd).float() - q_want).abs().max().item() < 1.5e-2 * scale      # one rounding to bfloat16 less
    pa, pb = sa["pool"].float(), sb["pool"].float()
    assert torch.equal(torch.isnan(pa), torch.isnan(pb))                                # the same places written, no other
    if write_cache:
        pa, pb = torch.nan_to_num(pa), torch.nan_to_num(pb)
        assert (pb[:, 0] - pa[:, 0][..., order]).abs().max().item() < 1.5e-2 * pa[:, 0].abs().max().item()
        assert torch.equal(pb[:, 1], pa[:, 1])
    k.check_status("cuda")


@pytest.mark.parametrize("dtype,hd,table_len", [(torch.float32, 24, 0), (torch.bfloat16, 64, 0), (torch.bfloat16, 64, 256)])
def test_rope_append_skips_rows_of_no_sequence(dtype, hd, table_len):
    """Rows with sequence index -1 (padding up to a captured graph's size) write nothing to the cache: the
    pool after a padded call equals the pool after the call without the padding (both rope kernels)."""
    k = K()
    H, KV = 3, 2
    lens_before, lens_new = [0, 70], [9, 66]
    n, pad = sum(lens_new), 11
    inv_freq = torch.tensor([1e4 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64, device="cuda")
    table = k.rope_table(inv_freq, table_len) if table_len else None
    g = torch.Generator(device="cuda").manual_seed(hd)
    qkv = torch.randn(n + pad, (H + 2 * KV) * hd, device="cuda", generator=g).to(dtype)
    sa = paged_setup(lens_before, lens_new, KV, hd, dtype, seed=3)
    sb = paged_setup(lens_before, lens_new, KV, hd, dtype, seed=3)
    a, b = qkv[:n].clone(), qkv.clone()
    minus = torch.full((pad,), -1, dtype=torch.int32, device="cuda")
    zeros = torch.zeros(pad, dtype=torch.int32, device="cuda")
    mp = max(x + y for x, y in zip(lens_before, lens_new)) - 1
    k.rope_append(a, sa["token_seq"], sa["token_pos"], sa["slots"], sa["table"], inv_freq, hd, False, sa["pool"], H, KV, hd,
                  table=table, max_position=mp)
    k.rope_append(b, torch.cat([sb["token_seq"], minus]), torch.cat([sb["token_pos"], zeros]), sb["slots"], sb["table"],
                  inv_freq, hd, False, sb["pool"], H, KV, hd, table=table, max_position=mp)
    assert torch.equal(a, b[:n])
    pa, pb = sa["pool"].float(), sb["pool"].float()
    assert torch.equal(torch.isnan(pa), torch.isnan(pb))
    assert torch.equal(torch.nan_to_num(pa), torch.nan_to_num(pb))


def test_gemv_rotary_epilogue_skips_rows_of_no_sequence():
    k = K()
    n, H, KV, hd, width = 6, 4, 2, 64, 256
    g = torch.Generator(device="cuda").manual_seed(77)
    w = (torch.randn((H + 2 * KV) * hd, width, device="cuda", generator=g) * 0.08).to(torch.bfloat16)
    x = torch.randn(n, width, device="cuda", generator=g).to(torch.bfloat16)
    lens_before = [5 + 37 * i for i in range(n)]
    inv_freq = torch.tensor([5e5 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64, device="cuda")
    table = k.rope_table(inv_freq, max(lens_before) + 2)
    pools = []
    for skipped in ((), (1, 4)):
        st = paged_setup(lens_before, [1] * n, KV, hd, torch.bfloat16, seed=5)
        seq = st["token_seq"].clone()
        for i in skipped:
            seq[i] = -1
        q = torch.empty((n, H * hd), device="cuda", dtype=torch.bfloat16)
        rope = dict(token_pos=st["token_pos"], token_seq=seq, slot_of_seq=st["slots"], block_table=st["table"], table=table,
                    pool=st["pool"], n_heads=H, n_kv=KV, head_dim=hd, write_cache=True, max_position=max(lens_before))
        k.gemv(w, n, x=x, out=q, rope=rope)
        pools.append((st, st["pool"].float()))
    (st, full), (_, part) = pools
    for s in range(n):          # sequence s holds one new token at position lens_before[s]
        page = int(st["host_table"][st["host_slots"][s], lens_before[s] // k.PAGE])
        entry_full, entry_part = full[page, :, :, lens_before[s] % k.PAGE], part[page, :, :, lens_before[s] % k.PAGE]
        assert not torch.isnan(entry_full).any()
        if s in (1, 4):
            assert torch.isnan(entry_part).all()
        else:
            assert torch.equal(entry_full, entry_part)
    k.check_status("cuda")


def test_gemv_refuses_what_it_cannot_do():
    k = K()
    assert not k.gemv_supported(17, 10, 64) and not k.gemv_supported(4, 10, 96)
    w = torch.zeros(16, 96, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(k.KernelError, match="multiple of 64"):
        k.gemv(w, 1, x=torch.zeros(1, 96, device="cuda", dtype=torch.bfloat16), out=torch.zeros(1, 16, device="cuda"))


@pytest.mark.parametrize("H,KV,hd", [(32, 8, 64), (8, 8, 64), (16, 2, 128), (4, 2, 128), (24, 8, 128), (12, 2, 64), (5, 1, 64), (7, 1, 128)])
@pytest.mark.parametrize("n_splits", [1, 4, 11])
def test_decode_attention_specialised_equals_general(H, KV, hd, n_splits):
    """The specialised decode kernel and the general kernel on the same cache, and both against the
    plain restatement (through run_attention_case)."""
    run_attention_case(torch.bfloat16, H, KV, hd, [0, 63, 64, 700, 129, 15], [1] * 6, 0, n_splits, seed=21)
    run_attention_case(torch.bfloat16, H, KV, hd, [300, 64, 5], [1] * 3, 100, n_splits, seed=22)


def test_rope_table_equals_on_the_fly():
    k = K()
    H, KV, hd = 4, 2, 64
    st = paged_setup([0, 100], [90, 30], KV, hd, torch.bfloat16, seed=30)
    inv_freq = torch.tensor([5e5 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(31)
    qkv = torch.randn(120, (H + 2 * KV) * hd, device="cuda", generator=g).to(torch.bfloat16)
    a, b = qkv.clone(), qkv.clone()
    pool_b = st["pool"].clone()
    k.rope_append(a, st["token_seq"], st["token_pos"], st["slots"], st["table"], inv_freq, hd, False, st["pool"], H, KV, hd)
    table = k.rope_table(inv_freq, 110)          # covers some positions, not all
    k.rope_append(b, st["token_seq"], st["token_pos"], st["slots"], st["table"], inv_freq, hd, False, pool_b, H, KV, hd, table=table)
    assert torch.equal(a, b)
    assert torch.equal(torch.nan_to_num(st["pool"].float()), torch.nan_to_num(pool_b.float()))
    # a table that covers the whole step: the vector kernel (same numbers up to the last bit of a product)
    c, pool_c = qkv.clone(), torch.full_like(st["pool"], float("nan"))
    full = k.rope_table(inv_freq, 256)
    k.rope_append(c, st["token_seq"], st["token_pos"], st["slots"], st["table"], inv_freq, hd, False, pool_c, H, KV, hd,
                  table=full, max_position=129)
    torch.testing.assert_close(c.float(), a.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(torch.nan_to_num(pool_c.float()), torch.nan_to_num(st["pool"].float()), rtol=1e-2, atol=1e-2)
    assert torch.equal(torch.isnan(pool_c.float()), torch.isnan(st["pool"].float()))


def test_argmax_large_vocabulary():
    g = torch.Generator(device="cuda").manual_seed(40)
    logits = torch.randn(9, 128256, device="cuda", generator=g)
    logits[3, 100000] = logits[3, 5000] = 30.0       # a tie across chunks: the lower index
    logits[4, 128255] = 31.0
    out = torch.empty(9, device="cuda", dtype=torch.int32)
    K().argmax(logits, out)
    want = logits.argmax(-1)
    want[3] = 5000
    assert out.tolist() == want.tolist()


@pytest.mark.parametrize("vocab,rows", [(128256, 9), (20000, 70), (1000, 5)])
def test_argmax_in_one_launch_feeds_the_next_step(vocab, rows):
    """With tickets a large vocabulary's argmax is one launch (the block that finishes a row's last chunk merges the
    row) and gives what the two launches give, planted ties across chunks included, the tickets zero again; with
    `advance` the same launch makes the step feed itself: tokens, positions, the run's history and its step counter
    over several steps, as the separate kernel does (which a small vocabulary still takes)."""
    g = torch.Generator(device="cuda").manual_seed(42)
    tickets = torch.zeros(rows + 1, device="cuda", dtype=torch.int32)
    tokens = torch.zeros(rows, device="cuda", dtype=torch.int32)
    pos = torch.arange(rows, device="cuda", dtype=torch.int32) * 7
    history = torch.full((3, rows), -1, device="cuda", dtype=torch.int32)
    step_no = torch.zeros(1, device="cuda", dtype=torch.int32)
    want_history = []
    for step in range(4):            # one more than the history holds: the last is not recorded
        logits = torch.randn(rows, vocab, device="cuda", generator=g)
        logits[1, vocab - 1] = logits[1, 17] = 40.0                   # a tie across chunks: the lower index
        logits[2, vocab - 1] = 41.0
        want = logits.argmax(-1)
        want[1] = 17
        two = torch.empty(rows, device="cuda", dtype=torch.int32)
        K().argmax(logits, two)
        one = torch.empty(rows, device="cuda", dtype=torch.int32)
        K().argmax(logits, one, tickets=tickets)
        assert two.tolist() == want.tolist() and one.tolist() == want.tolist()
        fed = torch.empty(rows, device="cuda", dtype=torch.int32)
        K().argmax(logits, fed, tickets=tickets, advance=(tokens, pos, history, step_no))
        want_history.append(want.tolist())
        assert fed.tolist() == want.tolist() and tokens.tolist() == want.tolist()
        assert pos.tolist() == [7 * r + step + 1 for r in range(rows)]
        assert step_no.item() == step + 1
        assert tickets.tolist() == [0] * (rows + 1)
    assert history.tolist() == want_history[:3]
    with pytest.raises(K().KernelError):
        K().argmax(logits, fed, tickets=tickets[:rows])


@pytest.mark.parametrize("vocab", [1000, 128256])
def test_argmax_and_sample_fill_a_pinned_mirror(vocab):
    """The sampling kernels write their results to pinned host memory as well when given a `mirror` (the captured
    decode step's way of handing tokens to a polling host): after the stream is done it holds what `out` holds,
    for the one-kernel argmax, the two-stage one and the draw; rows beyond the batch are left alone."""
    g = torch.Generator(device="cuda").manual_seed(41)
    logits = torch.randn(5, vocab, device="cuda", generator=g) * 3
    out = torch.empty(5, device="cuda", dtype=torch.int32)
    mirror = torch.full((7,), -1, dtype=torch.int32).pin_memory()
    K().argmax(logits, out, mirror=mirror)
    torch.cuda.synchronize()
    assert out.tolist() == logits.argmax(-1).tolist()
    assert mirror.tolist() == out.tolist() + [-1, -1]
    mirror.fill_(-1)
    f = torch.tensor([[0.8] * 5, [0.9] * 5], dtype=torch.float32, device="cuda")
    ids = torch.tensor([[7] * 5, [1, 2, 3, 4, 5]], dtype=torch.int64, device="cuda")
    counters = torch.arange(5, dtype=torch.int64, device="cuda")
    K().sample(logits, f[0], f[1], ids[0], ids[1], counters, out, mirror=mirror)
    torch.cuda.synchronize()
    plain = torch.empty(5, device="cuda", dtype=torch.int32)
    K().sample(logits, f[0], f[1], ids[0], ids[1], counters, plain)
    assert out.tolist() == plain.tolist()
    assert mirror.tolist() == out.tolist() + [-1, -1]
    with pytest.raises(K().KernelError):
        K().argmax(logits, out, mirror=torch.zeros(7, dtype=torch.int32))          # not pinned
    with pytest.raises(K().KernelError):
        K().argmax(logits, out, mirror=torch.zeros(3, dtype=torch.int32).pin_memory())   # too short


@pytest.mark.parametrize("H,KV,hd", [(8, 2, 64), (4, 4, 128), (6, 1, 64)])
def test_prompt_attention_on_tensor_cores(H, KV, hd):
    """Prompts of head size 64 / 128 in bfloat16 take the tensor-core kernel: whole prompts of unequal
    lengths, prompts that continue a cached prefix, and a window; each against the general kernel and
    against the plain restatement (through run_attention_case)."""
    run_attention_case(torch.bfloat16, H, KV, hd, [0, 0, 0, 0, 0], [16, 63, 64, 65, 333], 0, 1, seed=50)
    run_attention_case(torch.bfloat16, H, KV, hd, [10, 100, 64, 700], [17, 40, 128, 70], 0, 1, seed=51)
    run_attention_case(torch.bfloat16, H, KV, hd, [0, 130, 64], [200, 90, 31], 75, 1, seed=52)


@pytest.mark.parametrize("H,KV,hd", [(8, 2, 64), (6, 2, 128)])
def test_prompt_attention_over_thousands_of_keys(H, KV, hd):
    """Prompts of the lengths that are served: 4,096 tokens at once (64 pages: every ring of the kernel goes round
    many times, and the long blocks run beside short ones), long prompts that continue a long cached prefix, a
    batch of unequal prompts, and a window of a thousand keys; against the general kernel and the plain
    restatement."""
    run_attention_case(torch.bfloat16, H, KV, hd, [0], [4096], 0, 1, seed=80)
    run_attention_case(torch.bfloat16, H, KV, hd, [2000, 130, 0], [1500, 700, 333], 0, 1, seed=81)
    run_attention_case(torch.bfloat16, H, KV, hd, [1000, 0], [1100, 2100], 1000, 1, seed=82)


# (cached tokens, new tokens, window, positions of the planted key).  16 to 63 new tokens take the mma.sync prompt
# kernel in bfloat16, 64 and more the tcgen05 one.  Planted: the first key, the ends of pages (63, 64, 127, 128),
# the last cached key and the first new one, the last key of a partial page; with a window w, for a row at position
# pos the key pos - w must be ignored and pos - w + 1 must win, for the rows at both ends of a 128-row tile of the
# step (rows 0, 127, 128 and the last).
PLANTED = [
    (0, 40, 0, [0, 17, 39]),
    (70, 50, 0, [0, 63, 64, 69, 70, 100, 119]),
    (0, 200, 0, [0, 63, 64, 127, 128, 150, 199]),
    (130, 300, 0, [0, 63, 64, 127, 128, 129, 130, 257, 258, 383, 384, 429]),
    (200, 260, 75, [125, 126, 252, 253, 254, 384, 385, 459]),
    (0, 300, 128, [0, 1, 63, 64, 127, 128, 171, 172, 299]),
    (10, 50, 24, [0, 9, 10, 35, 36, 59]),
    (100, 33, 37, [63, 64, 95, 96, 100, 132]),
    # two dozen pages: the rings of key pages, value pages and score tiles go round several times before the planted
    # key makes a row move its reference maximum and rescale what it has summed
    (1000, 600, 0, [0, 640, 999, 1000, 1343, 1599]),
    (900, 700, 512, [388, 389, 900, 1087, 1088, 1599]),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,hd", [(4, 2, 64), (4, 1, 128)])
@pytest.mark.parametrize("before,new,window,planted", PLANTED)
def test_prompt_attention_finds_planted_keys(dtype, H, KV, hd, before, new, window, planted):
    """Random keys and values hide a lost key or a window edge that is off by one (the output moves by 1/n).
    Here all keys are tiny but one, which matches every query: a row that may see it must return that key's
    value, a row that may not (the key lies after it, or before its window) the mean of what it does see."""
    k = K()
    S = before + new
    scale = 1.0
    for target in planted:
        st = paged_setup([before], [new], KV, hd, dtype, seed=target)
        g = torch.Generator(device="cuda").manual_seed(70 + target)
        kh = (0.01 * torch.randn(S, KV, hd, device="cuda", generator=g)).to(dtype)
        vh = torch.randn(S, KV, hd, device="cuda", generator=g).to(dtype)
        kh[target] = 4.0
        write_history(st, [kh], [vh])
        q = torch.zeros(new, (H + 2 * KV) * hd, device="cuda", dtype=dtype)
        q[:, : H * hd] = 1.0
        out = torch.empty(new, H * hd, device="cuda", dtype=dtype)
        k.attention(q, q.shape[1], st["pool"], st["table"], st["cu"], st["slots"], st["starts"], out, new, 1, new,
                    H, KV, hd, scale, window=window, max_kv_len=S)
        k.check_status("cuda")
        want = attention_reference(q.double().view(new, -1, hd)[:, :H], kh.double(), vh.double(), before, scale, window)
        got = out.double().view(new, H, hd)
        assert not torch.isnan(got).any()
        bad = ((got - want).abs() > 2e-2 + 2e-2 * want.abs()).flatten(1).any(1)
        assert not bad.any(), (target, "first bad row", int(bad.nonzero()[0]), "of", new)
        # the rows that may see the planted key return its value
        pos = torch.arange(before, S, device="cuda")
        sees = (pos >= target) & ((pos - target < window) if window else torch.ones_like(pos, dtype=torch.bool))
        if sees.any():
            won = vh[target].double().repeat_interleave(H // KV, dim=0)
            assert (got[sees] - won).abs().max().item() < 2e-2


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (300, 520, 200), (77, 48, 1000), (2048, 3072, 2048), (513, 2048, 8192)])
def test_gemm_tc_store(m, n, k):
    """The tcgen05 product against fp64: exact bf16 products summed in fp32, rounded once to bf16."""
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    K().gemm_tc(x, w, out)
    K().check_status("cuda")
    want = x.double() @ w.double().T
    assert not torch.isnan(out.float()).any()
    assert (out.double() - want).abs().max().item() < 5e-3 * want.abs().max().item()


@pytest.mark.parametrize("m,inner,k", [(128, 128, 64), (333, 520, 192), (2048, 8192, 2048)])
def test_gemm_tc_gated(m, inner, k):
    g = torch.Generator(device="cuda").manual_seed(m + inner)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    wgu = (torch.randn(2 * inner, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)         # [gate; up]
    tiled = torch.stack([wgu[:inner].view(inner // 8, 8, k), wgu[inner:].view(inner // 8, 8, k)], dim=1).reshape(2 * inner, k).contiguous()
    out = torch.full((m, inner), float("nan"), device="cuda", dtype=torch.bfloat16)
    K().gemm_tc(x, tiled, out, swiglu=True)
    K().check_status("cuda")
    gu = x.double() @ wgu.double().T
    want = gu[:, :inner] / (1 + torch.exp(-gu[:, :inner])) * gu[:, inner:]
    assert not torch.isnan(out.float()).any()
    assert (out.double() - want).abs().max().item() < 1e-2 * want.abs().max().item()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 520, 200), (77, 48, 1000), (2048, 2048, 2048), (513, 2052, 512)])
def test_gemm_tc_adds_into_the_stream(m, n, k):
    """The tcgen05 product with the stream epilogue: an fp32 [M, N] matrix gets the product added in place, at
    sizes that are no multiples of the tiles (and a row length that is no multiple of four floats)."""
    k_ = K()
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    stream = torch.randn(m, n, device="cuda", generator=g)
    want = stream.double() + x.double() @ w.double().t()
    k_.gemm_tc(x, w, add_into=stream)
    k_.check_status("cuda")
    torch.testing.assert_close(stream.double(), want, rtol=1e-4, atol=1e-4 * (k ** 0.5))
    with pytest.raises(k_.KernelError):
        k_.gemm_tc(x, w, add_into=stream.to(torch.bfloat16))


def test_step_tables_and_their_users():
    """The page of every new token and the block table's rows by sequence, looked up once per step: the tables
    themselves, and the kernels that take them (the rotary epilogue of the skinny product, decode attention) give
    what they give without them."""
    k = K()
    H, KV, hd, width = 4, 2, 64, 256
    lens_before = [5, 63, 64, 300, 129, 700]
    n = len(lens_before)
    st = paged_setup(lens_before, [1] * n, KV, hd, torch.bfloat16, seed=41)
    seq = st["token_seq"].clone()
    seq[2] = -1                                     # a row of no sequence
    token_page, seq_table = k.step_tables(seq, st["token_pos"], st["slots"], st["table"], n)
    for i in range(n):
        slot = st["host_slots"][i]
        want = -1 if i == 2 else int(st["host_table"][slot, lens_before[i] // k.PAGE])
        assert int(token_page[i]) == want
        assert torch.equal(seq_table[i].cpu(), st["host_table"][slot])
    g = torch.Generator(device="cuda").manual_seed(42)
    w = (torch.randn((H + 2 * KV) * hd, width, device="cuda", generator=g) * 0.08).to(torch.bfloat16)
    x = torch.randn(n, width, device="cuda", generator=g).to(torch.bfloat16)
    inv_freq = torch.tensor([5e5 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64, device="cuda")
    table = k.rope_table(inv_freq, max(lens_before) + 2)
    pools, qs = [], []
    for tp in (None, token_page):
        s2 = paged_setup(lens_before, [1] * n, KV, hd, torch.bfloat16, seed=41)
        q = torch.empty((n, H * hd), device="cuda", dtype=torch.bfloat16)
        rope = dict(token_pos=s2["token_pos"], token_seq=seq, slot_of_seq=s2["slots"], block_table=s2["table"], table=table,
                    pool=s2["pool"], n_heads=H, n_kv=KV, head_dim=hd, write_cache=True, max_position=max(lens_before), token_page=tp)
        k.gemv(w, n, x=x, out=q, rope=rope)
        pools.append(s2["pool"].float())
        qs.append(q)
    assert torch.equal(qs[0], qs[1])
    assert torch.equal(torch.isnan(pools[0]), torch.isnan(pools[1])) and torch.equal(torch.nan_to_num(pools[0]), torch.nan_to_num(pools[1]))
    # decode attention over a cache with history, with and without the rows by sequence
    hist_k = [torch.randn(t, KV, hd, device="cuda", generator=g).to(torch.bfloat16) for t in st["total"]]
    hist_v = [torch.randn(t, KV, hd, device="cuda", generator=g).to(torch.bfloat16) for t in st["total"]]
    write_history(st, hist_k, hist_v)
    qkv = torch.randn(n, (H + 2 * KV) * hd, device="cuda", generator=g).to(torch.bfloat16)
    outs = []
    _, seq_table = k.step_tables(st["token_seq"], st["token_pos"], st["slots"], st["table"], n)
    for tab in (None, seq_table):
        out = torch.empty(n, H * hd, device="cuda", dtype=torch.bfloat16)
        k.attention(qkv, qkv.shape[1], st["pool"], st["table"], st["cu"], st["slots"], st["starts"], out, n, n, 1, H, KV, hd, 0.125,
                    max_kv_len=max(st["total"]), seq_table=tab)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    k.check_status("cuda")
