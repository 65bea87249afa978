"""The product for a few dozen tokens (tcgen05, K cut over a cluster's blocks, sums met through distributed
shared memory) alone against fp64 restatements, at sizes other than the engine's test models: every end it
fuses, every cluster size, token counts on both sides of its paddings, sizes that are no multiples of its tiles."""
import pytest
import torch

from test_gpu_kernels import paged_setup

pytestmark = pytest.mark.gpu


def K():
    from burn_lm_b200 import kernels
    return kernels


def rand(shape, gen, scale=1.0):
    return (torch.randn(*shape, device="cuda", generator=gen) * scale).to(torch.bfloat16)


# (M, K): 16 tiles of a long K (clusters of 8), 24 tiles (clusters of 4), one tile of a short K (no cluster),
# sizes that fill no tile, many tiles (no cluster), a K that is no multiple of 64
SHAPES = [(2048, 8192), (3072, 2048), (128, 64), (200, 192), (77, 1000), (16384, 512), (2048, 2048), (520, 4160), (4096, 14336)]


@pytest.mark.parametrize("n", [1, 16, 17, 32, 33, 50, 64, 65, 128])
@pytest.mark.parametrize("m,k", SHAPES)
def test_gemm_sk_store(n, m, k):
    g = torch.Generator(device="cuda").manual_seed(n * 1000 + m + k)
    w, x = rand((m, k), g, 0.05), rand((n, k), g)
    want = x.double() @ w.double().T
    scale = want.abs().max().item()
    out32 = torch.full((n, m), float("nan"), device="cuda")
    K().gemm_sk(w, x, out=out32)
    K().check_status("cuda")
    assert (out32.double() - want).abs().max().item() < 3e-5 * scale + 1e-6        # exact products summed in fp32
    out16 = torch.full((n, m), float("nan"), device="cuda", dtype=torch.bfloat16)
    K().gemm_sk(w, x, out=out16)
    assert (out16.double() - want).abs().max().item() < 5e-3 * scale
    if n > 17:      # a token's result does not depend on the other tokens of the step: the same bits among fewer
        few = torch.empty(17, m, device="cuda")
        K().gemm_sk(w, x[:17].contiguous(), out=few)
        assert torch.equal(few, out32[:17])
    K().check_status("cuda")


@pytest.mark.parametrize("n", [17, 40, 64, 100])
@pytest.mark.parametrize("inner,k", [(576, 192), (8192, 2048), (200 * 8, 320)])
def test_gemm_sk_gated(n, inner, k):
    g = torch.Generator(device="cuda").manual_seed(n + inner)
    x = rand((n, k), g)
    wgu = rand((2 * inner, k), g, 0.05)           # [gate; up]
    tiled = torch.stack([wgu[:inner].view(inner // 8, 8, k), wgu[inner:].view(inner // 8, 8, k)], dim=1).reshape(2 * inner, k).contiguous()
    out = torch.full((n, inner), float("nan"), device="cuda", dtype=torch.bfloat16)
    K().gemm_sk(tiled, x, out=out, swiglu=True)
    K().check_status("cuda")
    gu = x.double() @ wgu.double().T
    want = gu[:, :inner] / (1 + torch.exp(-gu[:, :inner])) * gu[:, inner:]
    assert not torch.isnan(out.float()).any()
    assert (out.double() - want).abs().max().item() < 1e-2 * want.abs().max().item()


@pytest.mark.parametrize("n", [17, 33, 64])
@pytest.mark.parametrize("gdt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,inner", [(192, 320), (2048, 8192), (200 * 16 + 8, 64)])
def test_gemm_sk_adds_into_the_stream_and_hands_the_next_norm_over(n, gdt, width, inner):
    k = K()
    g = torch.Generator(device="cuda").manual_seed(n + width)
    act = rand((n, inner), g)
    wd = rand((width, inner), g, 0.1)
    gamma = (1 + 0.1 * torch.randn(width, device="cuda", generator=g)).to(gdt)
    stream = torch.randn(n, width, device="cuda", generator=g) * 3
    stream[n // 2, 7] = 40.0           # one lane that dominates its row's sum of squares
    before = stream.clone()
    plain = stream.clone()
    k.gemm_sk(wd, act, add_into=plain)
    new = before.double() + act.double() @ wd.double().T
    assert (plain.double() - new).abs().max().item() < 3e-5 * new.abs().max().item()
    scaled = torch.full((n, width), float("nan"), device="cuda", dtype=torch.bfloat16)
    squares = torch.full(((width + 15) // 16, k.SK_SQUARES_ROWS), float("nan"), device="cuda")
    k.gemm_sk(wd, act, add_into=stream, hand_over=(gamma, scaled, squares))
    k.check_status("cuda")
    assert torch.equal(stream, plain)
    want_scaled = stream.double() * gamma.double()
    assert (scaled.double() - want_scaled).abs().max().item() <= 2 ** -8 * want_scaled.abs().max().item()
    ssq = (stream.double() ** 2).sum(-1)
    assert (squares[:, :n].double().sum(0) - ssq).abs().max().item() < 1e-5 * ssq.max().item()
    if width % 8:
        return
    # the consumer divides by the root mean square: it is the norm, up to bfloat16 rounding of the input
    eps = 1e-5
    w2 = rand((136, width), g, 0.1)
    out = torch.empty(n, 136, device="cuda")
    k.gemm_sk(w2, scaled, out=out, squares=squares, eps=eps)
    h = stream.double()
    rms = torch.sqrt((h * h).mean(-1, keepdim=True) + eps)
    want = (scaled.double() @ w2.double().T) / rms
    assert (out.double() - want).abs().max().item() < 1e-4 * want.abs().max().item()
    want_norm = (h / rms * gamma.double()) @ w2.double().T
    assert (out.double() - want_norm).abs().max().item() < 2e-2 * want_norm.abs().max().item()
    k.check_status("cuda")


@pytest.mark.parametrize("n", [17, 40, 64])
@pytest.mark.parametrize("H,KV,hd,width", [(4, 2, 64, 256), (3, 1, 32, 192), (6, 3, 128, 512), (32, 8, 64, 2048)])
@pytest.mark.parametrize("write_cache", [True, False])
def test_gemm_sk_rotary_epilogue(n, H, KV, hd, width, write_cache):
    """Rotates q and k and appends k and v in its epilogue, against the plain product followed by the rotary
    kernel; rows of no sequence (index -1) reach no cache."""
    k = K()
    g = torch.Generator(device="cuda").manual_seed(n * 7 + hd)
    heads = H + (2 * KV if write_cache else 0)
    w = rand((heads * hd, width), g, 0.08)
    x = rand((n, width), g)
    order = torch.tensor(k.tiled_pair_order(hd), device="cuda")
    dealt = w.clone().view(heads, hd, width)
    dealt[: H + (KV if write_cache else 0)] = dealt[: H + (KV if write_cache else 0)][:, order]
    dealt = dealt.reshape(heads * hd, width).contiguous()
    lens_before = [5 + 37 * i for i in range(n)]                 # one token per sequence
    inv_freq = torch.tensor([5e5 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64, device="cuda")
    table = k.rope_table(inv_freq, max(lens_before) + 2)
    sa = paged_setup(lens_before, [1] * n, KV, hd, torch.bfloat16, seed=5)
    sb = paged_setup(lens_before, [1] * n, KV, hd, torch.bfloat16, seed=5)
    skipped = (3, n - 1)
    seq_a, seq_b = sa["token_seq"].clone(), sb["token_seq"].clone()
    for i in skipped:
        seq_a[i] = -1
        seq_b[i] = -1
    qkv = (x.double() @ w.double().T).to(torch.bfloat16)
    k.rope_append(qkv, seq_a, sa["token_pos"], sa["slots"], sa["table"], inv_freq, hd, k.PAIRS_HALVES, sa["pool"], H,
                  KV if write_cache else 0, hd, write_cache=write_cache, table=table, max_position=max(lens_before))
    q_want = qkv[:, : H * hd].reshape(n, H, hd)[:, :, order].float()
    q = torch.full((n, H * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
    rope = dict(token_pos=sb["token_pos"], token_seq=seq_b, slot_of_seq=sb["slots"], block_table=sb["table"], table=table,
                pool=sb["pool"], n_heads=H, n_kv=KV, head_dim=hd, write_cache=write_cache, max_position=max(lens_before))
    k.gemm_sk(dealt, x, out=q, rope=rope)
    k.check_status("cuda")
    scale = q_want.abs().max().item()
    real = [i for i in range(n) if i not in skipped]       # what a row of no sequence holds afterwards is nobody's concern
    assert (q.view(n, H, hd).float()[real] - q_want[real]).abs().max().item() < 1.5e-2 * scale
    pa, pb = sa["pool"].float(), sb["pool"].float()
    assert torch.equal(torch.isnan(pa), torch.isnan(pb))                                # the same places written, no other
    if write_cache:
        pa, pb = torch.nan_to_num(pa), torch.nan_to_num(pb)
        assert (pb[:, 0] - pa[:, 0][..., order]).abs().max().item() < 1.5e-2 * pa[:, 0].abs().max().item()
        assert (pb[:, 1] - pa[:, 1]).abs().max().item() < 1e-2 * pa[:, 1].abs().max().item()


def test_gemm_sk_refuses_what_it_cannot_do():
    k = K()
    assert not k.gemm_sk_supported(129, 64, 64) and not k.gemm_sk_supported(8, 64, 60) and k.gemm_sk_supported(128, 1, 64)
    w = torch.zeros(16, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(k.KernelError, match="128 tokens"):
        k.gemm_sk(w, torch.zeros(200, 64, device="cuda", dtype=torch.bfloat16), out=torch.zeros(200, 16, device="cuda"))
