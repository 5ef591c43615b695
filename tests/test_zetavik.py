"""The Zetavik design in the engine, on the CPU with the plain stand-in kernels and on the GPU
with the CUDA kernels (``-m gpu``): same bodies.

Everything is compared with ``plain_zetavik`` (float64, token by token, one function per
mechanism).  The configurations are made here; they differ from each other in every size, in
the order of the layers, in the routing (groups or none, a shared expert or none, every expert
chosen), in whether a layer has a feed-forward, and one of them has sizes that no vector width
divides.
"""

import pytest
import torch

import fake_kernels
import helpers
import plain_zetavik as plain
import replay
from shiso_llm_b200 import LLM, SamplingParams
from shiso_llm_b200.cache import CacheManager
from shiso_llm_b200.config import ConfigMissing, InvalidValue, ZetavikConfig, plan_from_document
from shiso_llm_b200.engine.batch import StepBuilder, StepEntry
from shiso_llm_b200.parts import FEED_FORWARDS, MIXERS, NORMS, BuildEnv, FixedState, PagedKV, PartSpec
from shiso_llm_b200.weights import random_tensors
from shiso_llm_b200.weights.loader import target_dtype

BACKENDS = [pytest.param("cpu", id="plain-kernels-cpu"), pytest.param("cuda", id="cuda", marks=pytest.mark.gpu)]


def backend_args(backend):
    if backend == "cpu":
        return {"ops": fake_kernels, "device": "cpu"}
    return {"ops": None, "device": "cuda:0"}


def dtypes(backend):
    return ["float32"] if backend == "cpu" else ["float32", "bfloat16"]


def latent(heads, dim, rot, vdim, q_rank, kv_rank, scale, base=10000.0):
    return {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
            "rot": {"dims": rot, "base": base}}


def moe(experts, top, count, keep, scale, ff, shared):
    doc = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}
    if shared:
        doc["shared"] = {"ff": shared}
    return doc


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


DOC_A = {
    "architecture": "Zetavik", "vocab": 300, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        layer("lightning", {"heads": 2, "dim": 12, "vdim": 8, "decay": [0.9, 0.995]}, moe(6, 2, 3, 2, 1.5, 16, 24)),
        layer("latent_attention", latent(3, 8, 4, 6, 12, 20, 0.3), {"kind": "dense", "ff": 64}),
        layer("mamba2", {"heads": 4, "vdim": 6, "state": 10, "groups": 2, "conv": 3, "norm_groups": 3}, None),
        layer("latent_attention", latent(2, 4, 8, 10, 16, 24, 0.2, 100.0), moe(6, 2, 3, 2, 1.5, 16, 24)),
    ],
}

DOC_B = {
    "architecture": "Zetavik", "vocab": 211, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        layer("mamba2", {"heads": 2, "vdim": 16, "state": 16, "groups": 1, "conv": 4, "norm_groups": 1}, moe(4, 1, 1, 1, 1.0, 24, None)),
        layer("latent_attention", latent(5, 16, 8, 16, 24, 32, 0.25), None),
        layer("lightning", {"heads": 1, "dim": 20, "vdim": 36, "decay": [1.0]}, {"kind": "dense", "ff": 96}),
        layer("mamba2", {"heads": 6, "vdim": 8, "state": 24, "groups": 3, "conv": 2, "norm_groups": 4}, {"kind": "dense", "ff": 32}),
    ],
}

# sizes that no vector width divides: an odd width and vocabulary, heads of 6, 7 and 5, every expert chosen
DOC_C = {
    "architecture": "Zetavik", "vocab": 333, "width": 50, "norm": {"eps": 1e-5},
    "layers": [
        layer("latent_attention", latent(3, 6, 2, 7, 9, 11, 0.5, 7.0), moe(5, 5, 5, 5, 0.5, 6, 10)),
        layer("mamba2", {"heads": 3, "vdim": 5, "state": 7, "groups": 3, "conv": 5, "norm_groups": 5}, {"kind": "dense", "ff": 22}),
        layer("lightning", {"heads": 3, "dim": 6, "vdim": 9, "decay": [0.75, 0.9375, 0.998]}, moe(9, 3, 3, 1, 2.0, 10, None)),
    ],
}

DOCS = {"A": (DOC_A, 3), "B": (DOC_B, 4), "C": (DOC_C, 5)}


CLOSE_CALL = 0.05  # a choice of the router that a tenth of the score at stake would have turned


def check_rows(got, ref, dtype, what):
    """Per-row error against the plain logits, relative to their spread.  float32: sums in another
    order, rsqrtf/expf/sincosf and recurrences carried in float32 stay below 1e-4 of the spread;
    bfloat16: matrices, activations and the cache rounded to 8 bits of mantissa through a few
    layers stay below a tenth.  A wrong key, state, page or expert moves a row by the spread itself.
    ``ref`` may carry ``margin`` (per row, the router's closest call over all layers): in bfloat16 a
    row whose choice of experts hung on less than CLOSE_CALL of a score may choose otherwise, and is
    held to finiteness and half the spread only - no test rests on a close call."""
    margin = getattr(ref, "margin", None)
    got, ref = got.double(), ref.double()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    spread = ref.std().item()
    rms = (got - ref).pow(2).mean(-1).sqrt() / spread
    bound = 1e-4 if dtype == "float32" else 0.1
    if dtype != "float32" and margin is not None:
        close_call = margin < CLOSE_CALL
        assert rms[close_call].numel() == 0 or rms[close_call].max().item() <= 0.5, f"{what}: a row with a close call is off by more than half the spread"
        # a row after a close call carries a trace of it (its state and keys hold the other expert's output): twice the bound
        after = torch.cumsum(close_call.long(), 0) > 0
        rms = torch.where(close_call, torch.zeros_like(rms), torch.where(after, rms / 2, rms))
    worst = int(rms.argmax())
    assert rms.max().item() <= bound, f"{what}: row {worst} differs by {rms.max().item():.3e} of the spread (> {bound})"


class Reference(torch.Tensor):
    """Plain logits that remember the router's closest call of every row."""


def reference_logits(doc, tensors, tokens):
    margins = []
    logits = plain.forward(doc, dict(tensors), tokens, margins=margins)
    out = logits.as_subclass(Reference)
    out.margin = torch.stack(margins).min(0).values if margins else None
    return out


# --------------------------------------------------------------------------- configuration


def test_configuration_is_read_from_its_own_keys():
    arch, config, plan = plan_from_document(DOC_A)
    assert arch.name == "Zetavik" and isinstance(config, ZetavikConfig)
    assert (config.vocab, config.width, config.eps) == (300, 48, 1e-5)
    assert config.to_dict() == DOC_A and ZetavikConfig.from_dict(config.to_dict()) == config
    assert [l.mixer.kind for l in plan.layers] == ["lightning_attention", "latent_attention", "mamba2", "latent_attention"]
    assert [l.feed_forward.kind if l.feed_forward else None for l in plan.layers] == ["routed_experts", "relu2_ff", None, "routed_experts"]
    assert all(l.block.kind == "parallel_pre_norm" and l.feed_forward_norm is None for l in plan.layers)
    assert plan.head.params["tied_to"] == "embed" and plan.final_norm.kind == "layernorm"
    names = {s.name for s in helpers.tensor_specs_of(DOC_A)}
    assert {"embed", "final.norm", "l0.norm1", "l0.mix.q", "l0.mix.norm", "l0.mlp.router", "l0.mlp.e5.down", "l0.mlp.shared.gate",
            "l1.mix.dq", "l1.mix.dq.norm", "l1.mix.uq", "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv", "l1.mix.g",
            "l1.mlp.up", "l2.mix.in", "l2.mix.conv", "l2.mix.conv.b", "l2.mix.dt_bias", "l2.mix.A_log", "l2.mix.D"} <= names
    assert not any(n.startswith("l2.mlp") for n in names) and "head" not in names
    shapes = {s.name: s.shape for s in helpers.tensor_specs_of(DOC_A)}
    assert shapes["l2.mix.in"] == (2 * 24 + 2 * 2 * 10 + 4, 48) and shapes["l2.mix.conv"] == (24 + 40, 3)
    assert shapes["l1.mix.dkv"] == (24, 48) and shapes["l1.mix.uq"] == (3 * 12, 12) and shapes["l1.mix.g"] == (3, 48)


def test_configuration_refusals():
    def changed(path, value):
        import copy
        doc = copy.deepcopy(DOC_A)
        at = doc
        for key in path[:-1]:
            at = at[key]
        if value is None:
            del at[path[-1]]
        else:
            at[path[-1]] = value
        return doc

    with pytest.raises(ConfigMissing):
        ZetavikConfig.from_dict(changed(("norm",), None))
    with pytest.raises(ConfigMissing):
        ZetavikConfig.from_dict(changed(("layers", 1, "mixer", "kv_rank"), None))
    for path, value in [
        (("layers", 0, "type"), "conv"), (("layers", 0, "mixer", "decay"), [0.5]), (("layers", 2, "mixer", "groups"), 3),
        (("layers", 2, "mixer", "norm_groups"), 5), (("layers", 2, "mixer", "conv"), 1), (("layers", 1, "mixer", "rot", "dims"), 3),
        (("layers", 0, "mlp", "router", "top"), 7), (("layers", 0, "mlp", "router", "groups", "count"), 4),
        (("layers", 0, "mlp", "router", "groups", "keep"), 4), (("layers", 1, "mlp", "kind"), "glu"), (("vocab",), 0),
    ]:
        with pytest.raises(InvalidValue):
            ZetavikConfig.from_dict(changed(path, value))
    import copy
    few = copy.deepcopy(DOC_A)
    few["layers"][0]["mlp"]["router"].update(top=3, groups={"count": 3, "keep": 1})  # one group of two experts for three choices
    with pytest.raises(InvalidValue):
        ZetavikConfig.from_dict(few)


def test_cache_needs_of_the_three_mixers():
    _, _, plan = plan_from_document(DOC_A)
    env = BuildEnv(dtype=torch.float32, device=torch.device("cpu"), ops=fake_kernels)
    from shiso_llm_b200.parts import Model
    needs = Model(plan, env).cache_needs()
    assert needs[0] == FixedState((2, 12, 8))
    assert needs[1] == PagedKV(1, 24, None, 0) and needs[1].value_dim == 0  # one row [latent | shared key part], no value rows
    assert needs[2] == (FixedState((2, 64)), FixedState((4, 10, 6)))
    assert needs[3] == PagedKV(1, 32, None, 0)


# --------------------------------------------------------------------------- the whole model, every cut


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_every_cut_matches_the_plain_implementation(tmp_path, backend, name):
    doc, seed = DOCS[name]
    tensors = helpers.make_folder(tmp_path, doc, seed, std=0.15)
    lengths = [70, 40, 7, 33, 1]
    requests = {f"r{i}": helpers.random_prompt(n, doc["vocab"], 20 + i) for i, n in enumerate(lengths)}
    reference = {rid: reference_logits(doc, tensors, toks) for rid, toks in requests.items()}
    for dtype in dtypes(backend):
        engine = helpers.make_engine(tmp_path, dtype, page_size=4, kv_cache_tokens=192, ctx=128,
                                     max_num_batched_tokens=128, **backend_args(backend))
        steps, expect = [], []
        for rid, toks in requests.items():
            steps += helpers.whole(f"w-{rid}", toks)
            expect.append((f"w-{rid}", rid))
        steps += helpers.tail_one_by_one("t-r0", requests["r0"], 40)
        steps += helpers.portions("p-r0", requests["r0"], [13, 2, 7, 1, 3])
        steps += helpers.portions("p-r1", requests["r1"], [5, 4, 1])
        steps += helpers.portions("p-r3", requests["r3"], [2])
        expect += [("t-r0", "r0"), ("p-r0", "r0"), ("p-r1", "r1"), ("p-r3", "r3")]
        steps += replay.mixed_trace({f"m-{k}": v for k, v in requests.items()}, 3, 192)
        expect += [(f"m-{rid}", rid) for rid in requests]
        steps += replay.mixed_trace({f"n-{k}": v for k, v in reversed(list(requests.items()))}, 8, 192, tail=3)
        expect += [(f"n-{rid}", rid) for rid in requests]
        rows = helpers.run_steps(engine, steps)  # (checks the cache's books after every step)
        for trace_id, rid in expect:
            got = replay.stack_rows(rows, trace_id, len(requests[rid]))
            check_rows(got, reference[rid], dtype, f"{name} {dtype} {trace_id}")
        assert engine.cache.free_pages()[0] == 48 and engine.cache.slots.free_slots == 4


@pytest.mark.parametrize("backend", BACKENDS)
def test_cuts_agree_with_each_other_far_more_closely(tmp_path, backend):
    """The same request whole, token by token and in portions: the recurrences walk tokens in
    order and the attention folds keys in runs from position 0, so cuts agree to rounding."""
    doc, seed = DOCS["A"]
    helpers.make_folder(tmp_path, doc, seed, std=0.15)
    toks = helpers.random_prompt(90, doc["vocab"], 77)
    for dtype in dtypes(backend):
        engine = helpers.make_engine(tmp_path, dtype, page_size=16, kv_cache_tokens=256, ctx=256, max_num_batched_tokens=256,
                                     **backend_args(backend))
        whole = replay.stack_rows(helpers.run_steps(engine, helpers.whole("a", toks)), "a", len(toks))
        single = replay.stack_rows(helpers.run_steps(engine, helpers.portions("b", toks, [1])), "b", len(toks))
        cut = replay.stack_rows(helpers.run_steps(engine, helpers.portions("c", toks, [5, 2, 31, 3])), "c", len(toks))
        bound = (1e-5 if dtype == "float32" else 0.05) * whole.std().item()
        assert (whole - single).abs().max().item() <= bound
        assert (whole - cut).abs().max().item() <= bound


@pytest.mark.parametrize("backend", BACKENDS)
def test_long_decoding_with_a_request_that_joins(tmp_path, backend):
    """300 tokens one by one after a short prompt, a second request joining half-way; the trace
    runs twice in one engine, so every page and slot is used again."""
    doc, seed = DOCS["B"]
    tensors = helpers.make_folder(tmp_path, doc, seed, std=0.15)
    a = helpers.random_prompt(330, doc["vocab"], 5)
    b = helpers.random_prompt(110, doc["vocab"], 6)
    reference = {"a": reference_logits(doc, tensors, a), "b": reference_logits(doc, tensors, b)}
    steps = [([("a", a[:30], list(range(30)))], [])]
    for i in range(30, 330):
        entries = [("a", [a[i]], [0])]
        j = i - 130  # b: a prompt of 20 at a's position 130, then one token a step
        if j == 0:
            entries.insert(0, ("b", b[:20], list(range(20))))
        elif 0 < j <= 90:
            entries.append(("b", [b[19 + j]], [0]))
        steps.append((entries, [r for r, n in (("a", 329), ("b", 220)) if i == n]))
    for dtype in dtypes(backend):
        engine = helpers.make_engine(tmp_path, dtype, page_size=8, kv_cache_tokens=456, ctx=336, max_num_batched_tokens=64,
                                     **backend_args(backend))
        helpers.run_steps(engine, steps[:150])
        engine.finish("a"), engine.finish("b")
        rows = helpers.run_steps(engine, steps)
        check_rows(replay.stack_rows(rows, "a", 330), reference["a"], dtype, f"long decoding {dtype}")
        check_rows(replay.stack_rows(rows, "b", 110), reference["b"], dtype, f"the request that joined {dtype}")
        assert engine.cache.free_pages()[0] == 57 and engine.cache.slots.free_slots == 4


DOC_WIDE = {
    "architecture": "Zetavik", "vocab": 400, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        layer("latent_attention", latent(6, 32, 16, 32, 48, 96, 0.15), moe(8, 3, 4, 2, 1.0, 48, 64)),
        layer("lightning", {"heads": 2, "dim": 64, "vdim": 96, "decay": [0.97, 0.999]}, {"kind": "dense", "ff": 160}),
        layer("mamba2", {"heads": 4, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 2}, moe(8, 3, 4, 2, 1.0, 48, 64)),
    ],
}


@pytest.mark.gpu
def test_long_portions_and_wide_heads(tmp_path):
    """Heads and states of real widths, a 700-token request: whole, in long and short portions,
    with a second request in the batch, and the last tokens decoded at a context where a decode
    step's keys are shared out over several CTAs."""
    tensors = helpers.make_folder(tmp_path, DOC_WIDE, 9, std=0.08)
    a = helpers.random_prompt(700, DOC_WIDE["vocab"], 1)
    b = helpers.random_prompt(150, DOC_WIDE["vocab"], 2)
    reference = {"a": reference_logits(DOC_WIDE, tensors, a), "b": reference_logits(DOC_WIDE, tensors, b)}
    for dtype in ("bfloat16", "float32"):
        engine = helpers.make_engine(tmp_path, dtype, page_size=16, kv_cache_tokens=4096, ctx=2048, max_num_batched_tokens=1024)
        rows = helpers.run_steps(engine, helpers.whole("w", a))
        check_rows(replay.stack_rows(rows, "w", 700), reference["a"], dtype, f"one long portion {dtype}")
        rows = helpers.run_steps(engine, helpers.portions("p", a, [300, 100, 260, 1, 39]))
        check_rows(replay.stack_rows(rows, "p", 700), reference["a"], dtype, f"long and short portions {dtype}")
        rows = helpers.run_steps(engine, helpers.tail_one_by_one("t", a, 24))
        check_rows(replay.stack_rows(rows, "t", 700), reference["a"], dtype, f"decoded at a long context {dtype}")
        steps = [([("a", a[:400], list(range(400))), ("b", b[:5], list(range(5)))], []),
                 ([("b", b[5:6], [0]), ("a", a[400:], list(range(300)))], ["a"]),
                 ([("b", b[6:], list(range(144)))], ["b"])]
        rows = helpers.run_steps(engine, steps)
        check_rows(replay.stack_rows(rows, "a", 700), reference["a"], dtype, f"a long portion in a batch {dtype}")
        check_rows(replay.stack_rows(rows, "b", 150), reference["b"], dtype, f"its neighbour {dtype}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_through_the_trace_runner(tmp_path, dtype):
    """``bin/trace_run`` in a process of its own over a pool that holds barely the live requests:
    whole, last tokens one by one, changing portions and a mixed trace, against the plain logits."""
    doc, seed = DOCS["C"]
    model_dir = tmp_path / "model"
    tensors = helpers.make_folder(model_dir, doc, seed, std=0.15)
    lengths = [70, 100, 40, 7, 33, 1]
    requests = {f"r{i}": helpers.random_prompt(n, doc["vocab"], 60 + i) for i, n in enumerate(lengths)}
    steps, expect = [], []
    for rid, toks in requests.items():
        steps += helpers.whole(f"w-{rid}", toks)
        expect.append((f"w-{rid}", rid))
    steps += helpers.tail_one_by_one("t-r1", requests["r1"], 32)
    steps += helpers.portions("p-r1", requests["r1"], [13, 2, 7, 64, 3])
    steps += helpers.portions("p-r0", requests["r0"], [2, 3, 1, 2, 5, 1, 1, 17])
    expect += [("t-r1", "r1"), ("p-r1", "r1"), ("p-r0", "r0")]
    steps += replay.mixed_trace({f"m-{k}": v for k, v in requests.items()}, 5, 320)
    expect += [(f"m-{rid}", rid) for rid in requests]
    rows = replay.run_trace_run(model_dir, dtype, steps, 320, tmp_path / "out", doc["vocab"])
    for trace_id, rid in expect:
        got = replay.stack_rows(rows, trace_id, len(requests[rid]))
        check_rows(got, reference_logits(doc, tensors, requests[rid]), dtype, f"{dtype} {trace_id}")


@pytest.mark.parametrize("backend", BACKENDS)
def test_greedy_generation_through_the_scheduler(tmp_path, backend):
    doc, seed = DOCS["B"]
    tensors = helpers.make_folder(tmp_path, doc, seed, std=0.15)
    prompts = [helpers.random_prompt(n, doc["vocab"], 40 + n) for n in (19, 3, 30)]
    new = 12

    def plain_greedy(prompt):
        seq = list(prompt)
        for _ in range(new):
            seq.append(int(reference_logits(doc, tensors, seq)[-1].argmax()))
        return seq[len(prompt):]

    want = [plain_greedy(p) for p in prompts]
    args = backend_args(backend)
    llm = LLM(str(tmp_path), dtype="float32", ctx=64, page_size=4, max_num_seqs=2, max_num_batched_tokens=16, prefill_chunk=7,
              ops=args["ops"], device=args["device"])
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=new, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    llm.engine.cache.check()
    assert llm.engine.cache.slots.free_slots == 2


# --------------------------------------------------------------------------- mechanisms alone


def build_env(backend, dtype):
    if backend == "cpu":
        return BuildEnv(dtype=dtype, device=torch.device("cpu"), ops=fake_kernels)
    from shiso_llm_b200.kernels import ops

    ops.require()
    return BuildEnv(dtype=dtype, device=torch.device("cuda:0"), ops=ops)


def bind(part, env, seed, std=0.2, changes=None):
    specs = part.tensor_specs()
    stored = random_tensors(specs, seed, std, "bfloat16", 0.1)
    for name, fn in (changes or {}).items():
        stored[name] = fn(stored[name].float()).to(torch.bfloat16)
    by = {s.name: s for s in specs}
    part.bind({k: v.to(env.device, target_dtype(by[k], v.dtype, env.dtype)) for k, v in stored.items()})
    return {k: v.double() for k, v in stored.items()}


class Feeder:
    """Feeds sequences through one mixer in steps, over a cache manager of its own."""

    def __init__(self, mixer, env, slots=3, pages=64, page=4):
        self.mixer, self.env = mixer, env
        self.cache = CacheManager([mixer.cache_spec()], page, pages, slots, env.dtype, env.device)
        self.builder = StepBuilder(self.cache, env.device, 1024, slots)

    def step(self, parts):
        """``parts``: list of (request, rows[n, hidden]); returns the mixer's output rows per request."""
        entries = [StepEntry(r, [0] * x.shape[0], []) for r, x in parts]
        starts = [self.cache.append(r, x.shape[0]) for r, x in parts]
        step = self.builder.build(entries, starts)
        x = torch.cat([x for _, x in parts]).to(self.env.device, self.env.dtype)
        y = self.mixer.forward(x, step, self.cache.view(0))
        y = (y.materialize() if hasattr(y, "materialize") else y).double().cpu()
        for r, _ in parts:
            self.cache.commit(r)
        self.cache.check()
        out, at = {}, 0
        for r, x in parts:
            out[r] = y[at : at + x.shape[0]]
            at += x.shape[0]
        return out


def close(got, want, dtype, what, loose=1.0):
    err = (got - want).abs().max().item()
    scale = want.abs().max().item()
    bound = (2e-5 if dtype == torch.float32 else 2.0 ** -5) * scale * loose
    assert err <= bound, f"{what}: {err:.3e} > {bound:.3e} (scale {scale:.3e})"


def mixer_dtypes(backend):
    return [torch.float32] if backend == "cpu" else [torch.float32, torch.bfloat16]


def plan_mixer(kind, mixer_doc, width, eps=1e-5):
    """The mixer's PartSpec as the plan builder makes it, with tensors named ``l0.mix.*``."""
    doc = {"architecture": "Zetavik", "vocab": 8, "width": width, "norm": {"eps": eps}, "layers": [layer(kind, mixer_doc, None)]}
    return plan_from_document(doc)[2].layers[0].mixer


def in_steps_and_batches(mixer, env, dtype, a, b, want_a, want_b, what, loose):
    """Two sequences through one mixer: a portion beside a single token, two tokens each in the other
    order, single tokens, the rests together; then a slot and pages that were given back."""
    feeder = Feeder(mixer, env)
    got_a, got_b = [], []
    out = feeder.step([("a", a[:20]), ("b", b[:1])])
    got_a.append(out["a"]); got_b.append(out["b"])
    out = feeder.step([("b", b[1:3]), ("a", a[20:22])])
    got_a.append(out["a"]); got_b.append(out["b"])
    for t in range(22, 27):
        got_a.append(feeder.step([("a", a[t : t + 1])])["a"])
    out = feeder.step([("a", a[27:]), ("b", b[3:])])
    got_a.append(out["a"]); got_b.append(out["b"])
    close(torch.cat(got_a), want_a, dtype, f"{what} a {dtype}", loose)
    close(torch.cat(got_b), want_b, dtype, f"{what} b {dtype}", loose)
    feeder.cache.release("a")
    again = feeder.step([("c", a[:5])])["c"]
    close(again, want_a[:5], dtype, f"{what} in a slot used again {dtype}", loose)


MAMBA = {"heads": 6, "vdim": 5, "state": 9, "groups": 3, "conv": 4, "norm_groups": 2}
LIGHTNING = {"heads": 3, "dim": 10, "vdim": 6, "decay": [0.5, 0.95, 1.0]}
LATENT = latent(5, 6, 4, 7, 10, 13, 0.4, 50.0)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind,mixer_doc,fn", [("mamba2", MAMBA, plain.mamba2), ("lightning", LIGHTNING, plain.lightning),
                                               ("latent_attention", LATENT, plain.latent_attention)])
def test_each_mixer_alone_in_steps_and_batches(backend, kind, mixer_doc, fn):
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        mixer = MIXERS.build(plan_mixer(kind, mixer_doc, 40), env)
        w = bind(mixer, env, 11)
        g = torch.Generator().manual_seed(1)
        a, b = torch.randn(37, 40, generator=g).to(dtype), torch.randn(9, 40, generator=g).to(dtype)
        want_a = fn(w, "l0.mix", mixer_doc, a.double(), 1e-5)
        want_b = fn(w, "l0.mix", mixer_doc, b.double(), 1e-5)
        in_steps_and_batches(mixer, env, dtype, a, b, want_a, want_b, kind, 4.0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_a_planted_key_far_back_and_at_page_borders(backend):
    """One key is made to stand out (its direction scaled up, and asked for by the last row), so that
    whether it is seen decides the output: the key sits at the sequence's first positions, far back
    among hundreds, on either side of page borders and of the runs of 32 keys the kernel works in,
    and right before the asking row; the asking row comes in a prompt's portion and as a decoded token."""
    dtype = torch.float32
    env = build_env(backend, dtype)
    doc = latent(2, 8, 4, 8, 12, 16, 1.0, 100.0)
    mixer = MIXERS.build(plan_mixer("latent_attention", doc, 32), env)
    w = bind(mixer, env, 31, 0.3)
    T = 300
    g = torch.Generator().manual_seed(3)
    base = torch.randn(T, 32, generator=g) * 0.1
    probe = torch.randn(32, generator=g)
    for planted in (0, 1, 3, 4, 31, 32, 150, 255, 256, 287, 288, 298):
        h = base.clone()
        h[planted] = probe * 3.0
        h[T - 1] = probe * 3.0  # the last row asks for it
        want = plain.latent_attention(w, "l0.mix", doc, h.double(), 1e-5)
        for tail in (0, 40):
            feeder = Feeder(mixer, env, pages=128)
            got = [feeder.step([("a", h[: T - tail - 7])])["a"], feeder.step([("a", h[T - tail - 7 : T - tail])])["a"]]
            for t in range(T - tail, T):
                got.append(feeder.step([("a", h[t : t + 1])])["a"])
            close(torch.cat(got), want, dtype, f"planted at {planted}, {tail} decoded", 2.0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_a_lost_state_or_convolution_window_shows(backend):
    """A recurrence whose decay is (nearly) one remembers its first token for ever, and a convolution
    reads the last rows of the portion before: the first token is made large, and portions of one to
    three rows follow each other, so that a state or a window that is dropped, zeroed or shifted at a
    portion's start changes every later output."""
    dtype = torch.float32
    env = build_env(backend, dtype)
    g = torch.Generator().manual_seed(8)
    h = torch.randn(60, 24, generator=g) * 0.3
    h[0] *= 10.0
    cuts = [1, 1, 2, 3, 1, 2, 5, 1, 1, 3, 7, 2, 1, 30]
    for kind, doc, fn, changes in [
        ("lightning", {"heads": 2, "dim": 6, "vdim": 4, "decay": [1.0, 0.999]}, plain.lightning, None),
        ("mamba2", {"heads": 2, "vdim": 4, "state": 6, "groups": 1, "conv": 4, "norm_groups": 1}, plain.mamba2,
         {"l0.mix.A_log": lambda t: t * 0 - 6.0}),  # exp(-exp(-6) dt): a decay within a per cent of one
    ]:
        mixer = MIXERS.build(plan_mixer(kind, doc, 24), env)
        w = bind(mixer, env, 5, 0.3, changes)
        want = fn(w, "l0.mix", doc, h.double(), 1e-5)
        feeder, got, at = Feeder(mixer, env), [], 0
        for n in cuts:
            got.append(feeder.step([("a", h[at : at + n])])["a"])
            at += n
        close(torch.cat(got), want, dtype, f"{kind} in short portions", 4.0)


def ff_part(mlp, width):
    doc = {"architecture": "Zetavik", "vocab": 8, "width": width, "norm": {"eps": 1e-5},
           "layers": [layer("lightning", {"heads": 1, "dim": 4, "vdim": 4, "decay": [0.5]}, mlp)]}
    return plan_from_document(doc)[2].layers[0].feed_forward


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("mlp", [{"kind": "dense", "ff": 50}, moe(10, 3, 5, 3, 1.75, 14, 20), moe(7, 2, 1, 1, 1.0, 9, None),
                                 moe(6, 6, 2, 2, 0.5, 8, 8), moe(8, 1, 8, 1, 1.0, 12, None)], ids=["dense", "groups", "plain", "all", "one"])
def test_feed_forwards_alone(backend, mlp):
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        part = FEED_FORWARDS.build(ff_part(mlp, 36), env)
        w = bind(part, env, 17, 0.3)
        g = torch.Generator().manual_seed(2)
        for rows in (1, 5, 70):
            h = torch.randn(rows, 36, generator=g).to(dtype)
            want = plain.dense_ff(w, "l0.mlp", h.double()) if mlp["kind"] == "dense" else plain.moe_ff(w, "l0.mlp", mlp, h.double())
            y = part.forward(h.to(env.device), None)
            y = (y.materialize() if hasattr(y, "materialize") else y).double().cpu()
            close(y, want, dtype, f"{mlp['kind']} feed-forward, {rows} rows {dtype}", 4.0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_group_limited_routing_on_made_up_scores(backend):
    """Scores chosen so that the group limit matters: the three best experts lie in three groups,
    of which two may stay - the third best expert is out although it beats everything in the kept groups."""
    env = build_env(backend, torch.float32)
    ops = env.ops
    logits = torch.full((2, 8), -5.0)
    logits[0, [0, 2, 4, 1]] = torch.tensor([3.0, 2.5, 2.0, 1.0])  # groups of two: {0,1} {2,3} {4,5} {6,7}
    logits[1, [7, 6, 0]] = torch.tensor([1.0, 0.9, 0.8])
    ids, weights = ops.moe_route(logits.to(env.device), 3, 4, 2, 2.0)
    scores = torch.softmax(logits.double(), -1)
    assert ids.cpu().tolist() == [[0, 2, 1], [7, 6, 0]]
    assert torch.allclose(weights.cpu().double(), 2.0 * torch.gather(scores, 1, ids.cpu().long()), rtol=1e-5)
    want = plain.route(scores, 3, 4, 2)
    assert want.nonzero()[:, 1].reshape(2, 3).tolist() == [[0, 1, 2], [0, 6, 7]]


@pytest.mark.parametrize("backend", BACKENDS)
def test_layer_norm_and_the_sum_of_two_block_outputs(backend):
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        norm = NORMS.build(PartSpec("layernorm", {"tensor": "n", "size": 50, "eps": 1e-5}), env)
        w = bind(norm, env, 3)
        g = torch.Generator().manual_seed(6)
        x = (torch.randn(9, 50, generator=g) * 3 + 2).to(env.device)
        d1, d2 = (torch.randn(9, 50, generator=g).to(env.device, dtype) for _ in range(2))
        want = plain.layer_norm(x.double().cpu(), w["n"], 1e-5)
        close(norm.apply(x.clone()).double().cpu(), want, dtype, "layer norm")
        total = x.double().cpu() + d1.double().cpu() + d2.double().cpu()
        residual = x.clone()
        got = norm.add_apply(residual, (d1, d2))
        close(got.double().cpu(), plain.layer_norm(total, w["n"], 1e-5), dtype, "sum of two + layer norm")
        assert (residual.double().cpu() - total).abs().max().item() <= 1e-5
        rows = torch.tensor([7, 2], dtype=torch.int32, device=env.device)
        residual = x.clone()
        got = norm.add_apply(residual, (d1,), rows)
        close(got.double().cpu(), plain.layer_norm((x.double().cpu() + d1.double().cpu())[[7, 2]], w["n"], 1e-5), dtype, "rows")
        assert torch.equal(residual, x)
