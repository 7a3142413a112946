"""GPU parity tests for variable-length causal prefill attention, through the C ABI, against
the CPU oracle's fp32-softmax result.  Tolerance: max-abs <= 2e-2, mean-abs <= 2e-3 (bf16)."""
import pytest
import torch

from aici_b200 import _lib, tch_cuda
import workloads
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


# The kernel has three shapes (aici_mha_varlen_fwd_shape): 1 = one query tile per CTA, two CTAs per
# SM (what sequences of up to 1024 keys get), 2 = two query tiles per CTA (longer ones), 3 = shape 2
# on CTA pairs with two-SM MMAs (never chosen automatically; group size a multiple of 4).  Every
# edge case below runs through the automatic choice and through each shape forced.
SHAPES = [pytest.param(0, id="auto"), pytest.param(1, id="one_tile"), pytest.param(2, id="two_tiles"),
          pytest.param(3, id="cta_pair")]


def _shape_fits(shape, hq, hkv):
    if shape == 3 and ((hq // hkv) % 4 != 0 or hq % 4 != 0):
        pytest.skip("the CTA-pair shape needs a group size that is a multiple of 4")


def _run(dev, w, causal=True, shape=0):
    _shape_fits(shape, w.q.shape[1], w.k.shape[1])
    return tch_cuda.flash_attn_varlen(w.q, w.k, w.v, w.cu_seqlens_q, w.cu_seqlens_k, w.max_seqlen_q,
                                      w.max_seqlen_k, w.scale, causal, shape=shape)


def _check_full(w, out, causal=True):
    want = O.flash_attn_varlen(w.q.cpu(), w.k.cpu(), w.v.cpu(), w.cu_seqlens_q.cpu(), w.cu_seqlens_k.cpu(),
                               w.max_seqlen_q, w.max_seqlen_k, w.scale, causal)
    got = out.cpu()
    assert not torch.isnan(got.float()).any()
    mx, mean = O.error_stats(got, want)
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)
    return want


@pytest.mark.parametrize("shape", SHAPES)
def test_config1_small_varlen(cuda_device, shape):
    w = workloads.prefill_small(cuda_device)
    out = _run(cuda_device, w, shape=shape)
    _check_full(w, out)
    assert _lib.last_status() == 0


@pytest.mark.parametrize("lens_q,lens_k,hq,hkv", [
    ([1, 127, 128, 129, 300], [1, 127, 128, 129, 300], 4, 4),   # ragged tails around the tile size
    ([5, 1, 40, 130], [70, 333, 40, 400], 8, 2),                # chunked prefill: k_len > q_len
    ([200, 40], [72, 8], 4, 1),                                 # k_len < q_len: leading rows see nothing
    ([512] * 3, [1536] * 3, 8, 2),                              # config-5 variant with 1024 cached tokens
])
@pytest.mark.parametrize("shape", SHAPES)
def test_ragged_and_bottom_right_mask(cuda_device, lens_q, lens_k, hq, hkv, shape):
    w = workloads.make_prefill("t", cuda_device, lens_q=lens_q, lens_k=lens_k, num_heads=hq,
                               num_kv_heads=hkv, seed=77)
    out = _run(cuda_device, w, shape=shape)
    want = _check_full(w, out)
    if lens_k[0] < lens_q[0]:
        assert float(out[:lens_q[0] - lens_k[0]].float().abs().max()) == 0.0
        assert float(want[:lens_q[0] - lens_k[0]].abs().max()) == 0.0
    assert _lib.last_status() == 0


@pytest.mark.parametrize("shape", SHAPES)
def test_non_causal(cuda_device, shape):
    w = workloads.make_prefill("t", cuda_device, lens_q=[100, 260], lens_k=[150, 260], num_heads=4,
                               num_kv_heads=2, seed=78)
    _check_full(w, _run(cuda_device, w, causal=False, shape=shape), causal=False)


def test_strided_inputs_from_fused_qkv(cuda_device):
    g = torch.Generator(device=cuda_device).manual_seed(79)
    n, hq, hkv, d = 333, 8, 2, 128
    qkv = workloads.randn_bf16((n, (hq + 2 * hkv) * d), cuda_device, g)
    q = qkv[:, :hq * d].view(n, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].view(n, hkv, d)
    v = qkv[:, (hq + hkv) * d:].view(n, hkv, d)
    cu = torch.tensor([0, 100, 333], dtype=torch.int32, device=cuda_device)
    out = tch_cuda.flash_attn_varlen(q, k, v, cu, cu, 233, 233, 0.09, True)
    want = O.flash_attn_varlen(q.cpu(), k.cpu(), v.cpu(), cu.cpu(), cu.cpu(), 233, 233, 0.09, True)
    mx, mean = O.error_stats(out.cpu(), want)
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)


@pytest.mark.parametrize("shape", SHAPES)
def test_large_scores_exercise_the_lazy_rescale(cuda_device, shape):
    """Scores that keep growing along the key axis force the running maximum to move by more
    than the rescale threshold many times."""
    n, hq = 1024, 2
    g = torch.Generator(device=cuda_device).manual_seed(80)
    q = workloads.randn_bf16((n, hq, 128), cuda_device, g)
    k = workloads.randn_bf16((n, hq, 128), cuda_device, g)
    v = workloads.randn_bf16((n, hq, 128), cuda_device, g)
    ramp = torch.linspace(0.2, 3.0, n, device=cuda_device).view(n, 1, 1)
    k = (k * ramp).to(torch.bfloat16)
    cu = torch.tensor([0, n], dtype=torch.int32, device=cuda_device)
    _shape_fits(shape, hq, hq)
    out = tch_cuda.flash_attn_varlen(q, k, v, cu, cu, n, n, 0.5, True, shape=shape)
    want = O.flash_attn_varlen(q.cpu(), k.cpu(), v.cpu(), cu.cpu(), cu.cpu(), n, n, 0.5, True)
    mx, mean = O.error_stats(out.cpu(), want)
    assert mx <= 4e-2 and mean <= MEAN_ABS, (mx, mean)  # peaked softmax: |out| up to ~4, bf16 ulp 1.6e-2


@pytest.mark.parametrize("shape", SHAPES)
def test_score_jump_beyond_the_single_pass_range(cuda_device, shape):
    """Keys of the last tiles are 8x larger: scores jump by far more than the range the single-pass
    softmax may absorb, so those tiles must be redone against their exact maximum (no inf/NaN)."""
    n, hq = 640, 2
    g = torch.Generator(device=cuda_device).manual_seed(82)
    q = workloads.randn_bf16((n, hq, 128), cuda_device, g)
    k = workloads.randn_bf16((n, hq, 128), cuda_device, g)
    v = workloads.randn_bf16((n, hq, 128), cuda_device, g)
    k[384:] = (k[384:].float() * 8).to(torch.bfloat16)
    k[600:] = (k[600:].float() * 4).to(torch.bfloat16)
    cu = torch.tensor([0, n], dtype=torch.int32, device=cuda_device)
    _shape_fits(shape, hq, hq)
    out = tch_cuda.flash_attn_varlen(q, k, v, cu, cu, n, n, 1.0, True, shape=shape)
    want = O.flash_attn_varlen(q.cpu(), k.cpu(), v.cpu(), cu.cpu(), cu.cpu(), n, n, 1.0, True)
    got = out.cpu().float()
    assert torch.isfinite(got).all()
    mx, mean = O.error_stats(got, want)
    assert mx <= 4e-2 and mean <= MEAN_ABS, (mx, mean)  # one-hot softmax rows: |out| up to ~4


@pytest.mark.parametrize("shape", SHAPES)
def test_mixed_step_prefill_chunks(cuda_device, shape):
    w = workloads.prefill_mixed_chunks(cuda_device)
    _check_full(w, _run(cuda_device, w, shape=shape))


@pytest.mark.parametrize("shape", [pytest.param(0, id="auto"), pytest.param(3, id="cta_pair")])
def test_long_context_sampled_rows(cuda_device, shape):
    """Config 4 shape at a length the CPU can check by rows: 2 x 8192, 64 q / 8 kv heads; all
    rows of the first and last query tile of each sequence for two heads plus random rows."""
    w = workloads.prefill_long(cuda_device, seqlen=8192)
    out = _run(cuda_device, w, shape=shape)
    torch.cuda.synchronize()
    assert _lib.last_status() == 0
    g = torch.Generator().manual_seed(81)
    rows = []
    for s in range(2):
        base = s * 8192
        for h in (0, 63):
            rows += [[s, base + r, h] for r in list(range(128)) + list(range(8192 - 128, 8192))]
    rnd_tok = torch.randint(0, 2 * 8192, (1024,), generator=g)
    rnd_head = torch.randint(0, 64, (1024,), generator=g)
    rows += [[int(t) // 8192, int(t), int(h)] for t, h in zip(rnd_tok, rnd_head)]
    rows = torch.tensor(rows, dtype=torch.int32)
    want = O.flash_attn_varlen_rows(w.q.cpu(), w.k.cpu(), w.v.cpu(), w.cu_seqlens_q.cpu(),
                                    w.cu_seqlens_k.cpu(), rows, w.scale, True)
    got = out.cpu()[rows[:, 1].long(), rows[:, 2].long()]
    mx, mean = O.error_stats(got, want)
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)


def test_config4_full_size_sampled_rows(cuda_device):
    """Config 4 at full size (2 x 32768, 64 q / 8 kv heads, 35 TFLOP): the CPU cannot evaluate it
    whole, so it checks, row by row in fp32, every row of the first and last query tile of each
    sequence for four heads (two kv groups) plus 4096 random (sequence, row, head) triples."""
    L = 32768
    w = workloads.prefill_long(cuda_device)
    assert w.q.shape[0] == 2 * L
    out = _run(cuda_device, w)
    torch.cuda.synchronize()
    assert _lib.last_status() == 0
    g = torch.Generator().manual_seed(82)
    rows = []
    for s in range(2):
        for h in (0, 7, 8, 63):
            rows += [[s, s * L + r, h] for r in list(range(128)) + list(range(L - 128, L))]
    rnd_tok = torch.randint(0, 2 * L, (4096,), generator=g)
    rnd_head = torch.randint(0, 64, (4096,), generator=g)
    rows += [[int(t) // L, int(t), int(h)] for t, h in zip(rnd_tok, rnd_head)]
    rows = torch.tensor(rows, dtype=torch.int32)
    want = O.flash_attn_varlen_rows(w.q.cpu(), w.k.cpu(), w.v.cpu(), w.cu_seqlens_q.cpu(),
                                    w.cu_seqlens_k.cpu(), rows, w.scale, True)
    got = out[rows[:, 1].long().to(cuda_device), rows[:, 2].long().to(cuda_device)].cpu()
    mx, mean = O.error_stats(got, want)
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)


@pytest.mark.parametrize("shape", SHAPES)
def test_neighbour_rows_behind_a_sequence_end_are_ignored(cuda_device, shape):
    """The last key/value tile of a packed sequence also holds the first rows of the next
    sequence; NaN/Inf there must not leak (the reference's loads are predicated)."""
    g = torch.Generator().manual_seed(93)
    lens = [100, 60, 200]
    total = sum(lens)
    q = torch.randn(total, 8, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(total, 2, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(total, 2, 128, generator=g).to(torch.bfloat16)
    cu = torch.tensor([0, 100, 160, 360], dtype=torch.int32)
    scale = 1.0 / 128 ** 0.5
    want = O.flash_attn_varlen(q, k, v, cu, cu, 200, 200, scale, True)
    kp, vp = k.clone(), v.clone()
    kp[100:160] = float("nan")   # poison the middle sequence: its own rows become NaN, its
    vp[100:160] = float("inf")   # neighbours must not notice
    out = tch_cuda.flash_attn_varlen(q.to(cuda_device), kp.to(cuda_device), vp.to(cuda_device),
                                     cu.to(cuda_device), cu.to(cuda_device), 200, 200, scale, True, shape=shape).cpu()
    keep = torch.cat([torch.arange(0, 100), torch.arange(160, 360)])
    assert torch.isfinite(out[keep].float()).all()
    mx, mean = O.error_stats(out[keep], want[keep])
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)


def test_rejects_unsupported(cuda_device):
    q = torch.zeros(4, 2, 128, dtype=torch.bfloat16, device=cuda_device)
    cu = torch.tensor([0, 4], dtype=torch.int32, device=cuda_device)
    with pytest.raises(_lib.AiciError, match="multiple of 4"):
        tch_cuda.flash_attn_varlen(q, q, q, cu, cu, 4, 4, 1.0, True, shape=3)
    with pytest.raises(_lib.AiciError, match="shape must be"):
        tch_cuda.flash_attn_varlen(q, q, q, cu, cu, 4, 4, 1.0, True, shape=4)
    q = torch.zeros(4, 2, 64, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(_lib.AiciError, match="head_size must be 128"):
        tch_cuda.flash_attn_varlen(q, q, q, cu, cu, 4, 4, 1.0, True)
    q = torch.zeros(4, 2, 128, dtype=torch.float16, device=cuda_device)
    with pytest.raises(_lib.AiciError, match="bf16"):
        tch_cuda.flash_attn_varlen(q, q, q, cu, cu, 4, 4, 1.0, True)
