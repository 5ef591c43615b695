"""The kernels of the Zetavik parts alone, each against the stand-in of the same name
(``fake_kernels``: float64, rounded once), at sizes other than any model's: both routes of the
latent attention (the general kernel, also with a decode step's keys shared out over CTAs, and the
tensor-core kernel of prompt portions), both routes of the per-head and per-expert products (CUDA
cores and tensor cores), the recurrence at every register layout, the convolution and its state."""

import pytest
import torch

import fake_kernels as fake
from test_kernels_gpu import close, make_step, ops, rnd

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def filled_latent_cache(step_cpu, table, page, pages, width, dtype, seed):
    """A cache whose rows for every position a sequence of the step can see are random."""
    cache = torch.zeros(pages, page, 1, width, dtype=dtype)
    g = torch.Generator().manual_seed(seed)
    flat = cache.view(-1, width)
    for s in range(step_cpu.num_seqs):
        last = int(step_cpu.start_pos[s]) + int(step_cpu.q_start[s + 1] - step_cpu.q_start[s])
        for p in range(last):
            flat[int(table[s, p // page]) * page + p % page] = (torch.randn(width, generator=g) * 0.5).to(dtype)
    return cache


@pytest.mark.parametrize("case", [
    # (heads, rank, width, page, q_lens, starts)
    (6, 112, 144, 16, [70, 1, 33], [0, 300, 17]),
    (5, 48, 64, 8, [16, 17, 1, 40], [0, 31, 64, 100]),
    (16, 224, 256, 16, [130], [515]),
    (3, 16, 32, 4, [9, 200], [1000, 0]),
])
def test_latent_attention_of_prompt_portions_on_both_routes(case):
    heads, rank, width, page, q_lens, starts = case
    t = ops()
    pages = sum(-(-(s + n) // page) for s, n in zip(starts, q_lens)) + 3
    cpu, gpu, table = make_step(q_lens, starts, page, pages, 5)
    cpu.max_q_len = gpu.max_q_len = max(q_lens)
    cpu.all_decode = gpu.all_decode = False
    gpu.h_q_start = cpu.q_start.tolist()
    cache = filled_latent_cache(cpu, table, page, pages, width, torch.bfloat16, 6)
    q = rnd((sum(q_lens), heads, width), torch.bfloat16, 7, 0.5)
    want = fake.latent_attention(q, rank, cache, table, page, 0.2, cpu)
    assert t.library().shiso_latent_prefill_supported(rank, width)
    for general in (False, True):
        got = t.latent_attention(q.cuda(), rank, cache.cuda(), table.cuda(), page, 0.2, gpu, general=general)
        close(got, want, torch.bfloat16, f"latent attention {case} general={general}")
    gpu.h_q_start = []  # a captured step: the tile count is a bound, not the sum
    got = t.latent_attention(q.cuda(), rank, cache.cuda(), table.cuda(), page, 0.2, gpu)
    close(got, want, torch.bfloat16, f"latent attention {case} with a bound of tiles")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", [(6, 112, 144, 16, 3000), (3, 11, 13, 4, 70), (16, 224, 256, 16, 2100), (4, 512, 576, 32, 1500)])
def test_latent_attention_of_single_tokens_with_shared_out_keys(dtype, case, monkeypatch):
    heads, rank, width, page, context = case
    t = ops()
    starts = [context - 1, 5, context // 2]
    pages = sum(-(-(s + 1) // page) for s in starts) + 3
    cpu, gpu, table = make_step([1, 1, 1], starts, page, pages, 9)
    cpu.all_decode = gpu.all_decode = True
    cache = filled_latent_cache(cpu, table, page, pages, width, dtype, 10)
    q = rnd((3, heads, width), dtype, 11, 0.5)
    want = fake.latent_attention(q, rank, cache, table, page, 0.3, cpu)
    for share_keys in (1 << 30, 256):  # one CTA a row and head group; or a share of the keys each
        monkeypatch.setattr(t, "LATENT_DECODE_SHARE_KEYS", share_keys)
        got = t.latent_attention(q.cuda(), rank, cache.cuda(), table.cuda(), page, 0.3, gpu)
        close(got, want, dtype, f"decode latent attention {case} {dtype} share {share_keys}", rel32=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_store_and_rotation(dtype):
    t = ops()
    rank, rot, page = 24, 8, 4
    q_lens, starts = [7, 1, 12], [3, 40, 0]
    cpu, gpu, table = make_step(q_lens, starts, page, 40, 12)
    rows = rnd((20, 50), dtype, 13)  # the latent row is a column range of a wider product
    w = rnd((rank,), torch.float32, 14).abs() + 0.5
    inv_freq = (100.0 ** (-torch.arange(rot // 2, dtype=torch.float64) * 2 / rot)).float()
    want = torch.zeros(40, page, 1, rank + rot, dtype=dtype)
    fake.latent_store(rows[:, 5 : 5 + rank + rot], rank, w, 1e-5, inv_freq, rot, cpu, want, table, page)
    got = torch.zeros(40, page, 1, rank + rot, dtype=dtype).cuda()
    t.latent_store(rows.cuda()[:, 5 : 5 + rank + rot], rank, w.cuda(), 1e-5, inv_freq.cuda(), rot, gpu, got, table.cuda(), page)
    close(got, want, dtype, f"latent store {dtype}", slack=1e-5)
    x = rnd((20, 3, 14), dtype, 15)
    want_r = torch.zeros(20, 3, 10, dtype=dtype)
    fake.rotate_heads(x[:, :, 4:], want_r, inv_freq, rot, cpu)
    wide = torch.zeros(20, 3, 16, dtype=dtype).cuda()
    t.rotate_heads(x.cuda()[:, :, 4:], wide[:, :, 6:], inv_freq.cuda(), rot, gpu)
    close(wide[:, :, 6:], want_r, dtype, f"rotate heads {dtype}", slack=1e-5)
    assert wide[:, :, :6].abs().max().item() == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(70, 5, 24, 40), (3, 2, 7, 9), (200, 16, 224, 64), (130, 8, 64, 224), (70, 2, 130, 456)])
def test_products_per_head(dtype, shape):
    tokens, heads, n, k = shape
    t = ops()
    wide = rnd((tokens, heads, k + 8), dtype, 1)
    w = rnd((heads, n, k), dtype, 2, 0.2)
    gate = rnd((tokens, heads + 3), dtype, 3)
    for g in (None, gate[:, 1 : 1 + heads]):
        want = torch.zeros(tokens, heads, n, dtype=dtype)
        fake.head_linear(wide[:, :, :k], w, want, gate=g)
        got = torch.zeros(tokens, heads, n + 8, dtype=dtype).cuda()
        t.head_linear(wide.cuda()[:, :, :k], w.cuda(), got[:, :, 8:], gate=None if g is None else gate.cuda()[:, 1 : 1 + heads])
        close(got[:, :, 8:], want, dtype, f"head_linear {shape} {dtype} gate={g is not None}", rel32=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(90, 40, 24, 6, 2), (5, 36, 10, 5, 5), (300, 128, 96, 8, 3), (1, 64, 32, 16, 4), (200, 520, 264, 4, 2)])
def test_routing_and_experts(dtype, shape):
    tokens, hidden, ff, experts, top = shape
    t = ops()
    x = rnd((tokens, hidden), dtype, 1)
    logits = rnd((tokens, experts), torch.float32, 2, 2.0)
    gate_up = rnd((experts, 2 * ff, hidden), dtype, 3, 0.2)
    down = rnd((experts, hidden, ff), dtype, 4, 0.2)
    extra = rnd((tokens, hidden), dtype, 5)
    ids, weights = t.moe_route(logits.cuda(), top, 1, 1, 1.5)
    want_ids, want_w = fake.moe_route(logits, top, 1, 1, 1.5)
    assert torch.equal(ids.cpu(), want_ids)
    close(weights, want_w, torch.float32, "weights", rel32=1e-5)
    ids_s, w_s = t.moe_route(logits.cuda(), 1, experts, 1, 1.0, sigmoid=True, renormalize=True)
    assert torch.equal(ids_s.cpu()[:, 0].long(), logits.argmax(-1)) and torch.allclose(w_s.cpu(), torch.ones(tokens, 1))
    for e in (None, extra):
        want = fake.routed_experts(x, want_ids, want_w, gate_up, down, e)
        got = t.routed_experts(x.cuda(), ids, weights, gate_up.cuda(), down.cuda(), None if e is None else e.cuda())
        close(got, want, dtype, f"experts {shape} {dtype}", rel32=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(3, 3, 10, 6), (4, 2, 16, 16), (6, 6, 40, 9), (2, 1, 64, 70), (4, 4, 128, 130), (2, 2, 200, 24)])
def test_recurrence_with_both_kinds_of_decay(dtype, shape):
    """Every register layout (16, 32, 64, 128 and 256 key rows), shared and own keys, long portions
    beside single tokens, a state that a step before left."""
    heads, groups, dim, vdim = shape
    t = ops()
    q_lens, starts = [37, 1, 2], [0, 9, 4]
    cpu, gpu, _ = make_step(q_lens, starts, 16, 8, 3, num_slots=5)
    T = sum(q_lens)
    q, k = rnd((T, groups * dim), dtype, 1, 0.3), rnd((T, groups * dim), dtype, 2, 0.3)
    v, dt = rnd((T, heads * vdim), dtype, 3), rnd((T, heads), dtype, 4)
    state = rnd((5, heads, dim, vdim), torch.float32, 5, 0.1)
    loss = (1.0 - torch.linspace(0.5, 1.0, heads, dtype=torch.float64)).float()
    a_log, dt_bias, skip = rnd((heads,), torch.float32, 6), rnd((heads,), torch.float32, 7), rnd((heads,), torch.float32, 8)
    for kind in ("fixed", "steps"):
        kw = {"silu_inputs": True, "head_loss": loss} if kind == "fixed" else {"dt": dt, "dt_bias": dt_bias, "a_log": a_log, "skip": skip}
        want_state = state.clone()
        want = fake.state_recurrence(q, k, v, want_state, cpu, heads, groups, dim, vdim, **kw)
        got_state = state.clone().cuda()
        got = t.state_recurrence(q.cuda(), k.cuda(), v.cuda(), got_state, gpu, heads, groups, dim, vdim,
                                 **{n: (x.cuda() if torch.is_tensor(x) else x) for n, x in kw.items()})
        close(got, want, torch.float32, f"recurrence {kind} {shape} {dtype}", rel32=2e-5)
        close(got_state, want_state, torch.float32, f"state {kind} {shape} {dtype}", rel32=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [2, 4, 7])
def test_causal_convolution_and_its_window(dtype, taps):
    t = ops()
    channels = 37
    q_lens, starts = [1, 30, 2, 3], [5, 0, 9, 2]  # portions shorter than, as long as, and longer than the window
    cpu, gpu, _ = make_step(q_lens, starts, 16, 8, 3, num_slots=6)
    x = rnd((36, channels + 5), dtype, 1)
    w, b = rnd((channels, taps), torch.float32, 2, 0.5), rnd((channels,), torch.float32, 3)
    state = rnd((6, taps - 1, channels), torch.float32, 4)
    want_state = state.clone()
    want = fake.causal_conv(x[:, 2 : 2 + channels], w, b, want_state, cpu)
    got_state = state.clone().cuda()
    got = t.causal_conv(x.cuda()[:, 2 : 2 + channels], w.cuda(), b.cuda(), got_state, gpu)
    close(got, want, dtype, f"causal conv {taps} {dtype}", rel32=1e-5)
    close(got_state, want_state, torch.float32, f"window {taps} {dtype}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_in_groups_with_both_gates(dtype):
    t = ops()
    x32, gate = rnd((9, 60), torch.float32, 1, 3.0), rnd((9, 70), dtype, 2)
    w = rnd((60,), torch.float32, 3).abs() + 0.5
    for groups, mode in ((1, None), (3, "silu_before"), (1, "sigmoid_after"), (5, "silu_before")):
        g = None if mode is None else gate[:, 4:64]
        want = fake.group_rmsnorm(x32, w, 1e-5, groups, dtype, gate=g, gate_mode=mode)
        got = t.group_rmsnorm(x32.cuda(), w.cuda(), 1e-5, groups, dtype, gate=None if g is None else gate.cuda()[:, 4:64], gate_mode=mode)
        close(got, want, dtype, f"group norm {groups} {mode} {dtype}", rel32=1e-5)
    xa = rnd((9, 70), dtype, 4)
    want = fake.group_rmsnorm(xa[:, 3:63], w, 1e-5, 2, dtype)
    close(t.group_rmsnorm(xa.cuda()[:, 3:63], w.cuda(), 1e-5, 2, dtype), want, dtype, f"group norm of activation rows {dtype}", rel32=1e-5)
