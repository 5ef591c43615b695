"""The Filulix design in the engine, on the CPU with the plain stand-in kernels and on the GPU
with the CUDA kernels (``-m gpu``): same bodies.

Everything is compared with ``plain_filulix`` (float64, token by token, one function per
mechanism).  The configurations are made here; they differ from each other in every size, in
the layer order, in the looped run, in the number of stream copies (one of them has a single
copy), in whether a layer has a feed-forward, and they use a pool size that is neither the
page size nor a divisor of the window.
"""

import pytest
import torch

import fake_kernels
import helpers
import plain_filulix as plain
import replay
from shiso_llm_b200 import LLM, SamplingParams
from shiso_llm_b200.cache import CacheManager
from shiso_llm_b200.config import ConfigMissing, FilulixConfig, InvalidValue, plan_from_document
from shiso_llm_b200.engine.batch import StepBuilder, StepEntry
from shiso_llm_b200.parts import MIXERS, BuildEnv, PartSpec
from shiso_llm_b200.weights import random_tensors
from shiso_llm_b200.weights.loader import target_dtype

BACKENDS = [pytest.param("cpu", id="plain-kernels-cpu"), pytest.param("cuda", id="cuda", marks=pytest.mark.gpu)]


def backend_args(backend):
    if backend == "cpu":
        return {"ops": fake_kernels, "device": "cpu"}
    return {"ops": None, "device": "cuda:0"}


def dtypes(backend):
    return ["float32"] if backend == "cpu" else ["float32", "bfloat16"]


def wkv_layer(heads, dim, rank, ff):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "rank": rank}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def parallel_layer(left, right, scales, ff):
    mixer = {"left": left, "right": right, "left_scale": scales[0], "right_scale": scales[1]}
    return {"type": "parallel", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


DOC_A = {
    "architecture": "Filulix", "vocab": 300, "width": 48, "streams": 3, "norm": {"eps": 1e-5},
    "embedding": {"scale": 2.5, "bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 7}},
    "layers": [
        wkv_layer(3, 16, 8, 64),
        parallel_layer(
            {"heads": 4, "kv_heads": 1, "dim": 8, "vdim": 12, "scale": 0.3, "mask": {"size": 9, "pool": 5}},
            {"heads": 2, "dim": 12, "vdim": 8, "decay": [0.9, 0.97], "rot": {"dims": 8, "base": 100.0}},
            (0.7, 1.3), None),
        wkv_layer(2, 24, 4, 80),
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}

DOC_B = {
    "architecture": "Filulix", "vocab": 211, "width": 64, "streams": 1, "norm": {"eps": 1e-6},
    "embedding": {"scale": 0.5, "bigram": {"buckets": 13, "mul_prev": 3, "mul_cur": 1000003}},
    "layers": [
        parallel_layer(
            {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.25, "mask": {"size": 16, "pool": 16}},
            {"heads": 4, "dim": 8, "vdim": 16, "decay": [0.5, 0.9, 0.99, 1.0], "rot": {"dims": 8, "base": 10000.0}},
            (1.0, 0.25), 96),
        wkv_layer(2, 32, 16, 96),
        parallel_layer(
            {"heads": 6, "kv_heads": 3, "dim": 4, "vdim": 20, "scale": 1.0, "mask": {"size": 3, "pool": 2}},
            {"heads": 1, "dim": 20, "vdim": 36, "decay": [0.8]},
            (0.5, 0.5), 32),
    ],
}

# sizes that no vector width divides: an odd width and vocabulary, head sizes of 10, 6 and 7, four copies
DOC_C = {
    "architecture": "Filulix", "vocab": 333, "width": 50, "streams": 4, "norm": {"eps": 1e-5},
    "embedding": {"scale": 7.0, "bigram": {"buckets": 50, "mul_prev": 1, "mul_cur": 1}},
    "layers": [
        wkv_layer(5, 10, 3, 30),
        parallel_layer(
            {"heads": 3, "kv_heads": 3, "dim": 6, "vdim": 7, "scale": 0.5, "mask": {"size": 20, "pool": 3}},
            {"heads": 3, "dim": 6, "vdim": 9, "decay": [0.75, 0.9375, 0.998], "rot": {"dims": 2, "base": 7.0}},
            (1.5, 0.75), 22),
    ],
    "loop": {"start": 0, "stop": 1, "times": 3},
}

DOCS = {"A": (DOC_A, 3), "B": (DOC_B, 4), "C": (DOC_C, 5)}


def check_rows(got, ref, dtype, what):
    """Per-row error against the plain logits, relative to their spread.  float32: sums in another
    order, rsqrtf/expf/sincosf and a recurrence carried in float32 stay below 1e-4 of the spread;
    bfloat16: matrices, activations and the cache rounded to 8 bits of mantissa through up to five
    layer runs stay below a tenth.  A wrong key, state or page moves a row by the spread itself."""
    got, ref = got.double(), ref.double()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    spread = ref.std().item()
    err = got - ref
    rms = err.pow(2).mean(-1).sqrt() / spread
    bound = 1e-4 if dtype == "float32" else 0.1
    worst = int(rms.argmax())
    assert rms.max().item() <= bound, f"{what}: row {worst} differs by {rms.max().item():.3e} of the spread (> {bound})"


def reference_logits(doc, tensors, tokens):
    return plain.forward(doc, {k: v for k, v in tensors.items()}, tokens)


# --------------------------------------------------------------------------- configuration


def test_configuration_is_read_from_its_own_keys():
    arch, config, plan = plan_from_document(DOC_A)
    assert arch.name == "Filulix" and isinstance(config, FilulixConfig)
    assert [e.layer for e in plan.order] == [0, 1, 2, 1, 2] == plain.run_order(DOC_A)
    assert [layer.mixer.kind for layer in plan.layers] == ["wkv_time_mix", "parallel_mixer", "wkv_time_mix"]
    assert plan.layers[1].feed_forward is None and "l1.norm2" in plan.unused_tensors
    assert plan.layers[0].block.kind == "hyper_pre_norm" and plan.layers[0].block.params["copies"] == 3
    again = FilulixConfig.from_dict(config.to_dict())
    assert again == config
    _, _, plan_b = plan_from_document(DOC_B)
    assert [e.layer for e in plan_b.order] == [0, 1, 2]
    plain_doc = {k: v for k, v in DOC_B.items() if k != "streams"}
    assert plan_from_document(plain_doc)[2].layers[0].block.kind == "pre_norm"


def test_configuration_refusals():
    def changed(path, value):
        import copy

        doc = copy.deepcopy(DOC_A)
        at = doc
        *head, last = path
        for key in head:
            at = at[key]
        if value is None:
            del at[last]
        else:
            at[last] = value
        return doc

    with pytest.raises(ConfigMissing):
        FilulixConfig.from_dict(changed(["width"], None))
    with pytest.raises(ConfigMissing):
        FilulixConfig.from_dict(changed(["layers", 1, "mixer", "left", "mask"], None))
    with pytest.raises(InvalidValue):
        FilulixConfig.from_dict(changed(["layers", 0, "type"], "conv"))
    with pytest.raises(InvalidValue):
        FilulixConfig.from_dict(changed(["layers", 1, "mixer", "right", "decay"], [0.5]))
    with pytest.raises(InvalidValue):
        FilulixConfig.from_dict(changed(["layers", 1, "mixer", "left", "kv_heads"], 3))
    with pytest.raises(InvalidValue):
        FilulixConfig.from_dict(changed(["loop"], {"start": 2, "stop": 1, "times": 2}))
    with pytest.raises(InvalidValue):
        FilulixConfig.from_dict(changed(["layers", 0, "mlp"], {"kind": "routed", "ff": 8}))


def test_cache_needs_of_composite_mixers_and_pooled_rows():
    _, _, plan = plan_from_document(DOC_A)
    from shiso_llm_b200.parts import Model
    from shiso_llm_b200.parts.base import FixedState, PagedKV

    model = Model(plan, BuildEnv(torch.float32, torch.device("cpu"), fake_kernels))
    needs = model.cache_needs()
    assert len(needs) == len(plan.order) + 1  # the embedding keeps the last token
    tokens, blocks, state = needs[1]
    assert isinstance(tokens, PagedKV) and tokens.window == 9 and tokens.every == 1 and tokens.value_dim == 12
    assert isinstance(blocks, PagedKV) and blocks.window is None and blocks.every == 5 and blocks.dtype == torch.float32
    assert isinstance(state, FixedState) and state.shape == (2, 12, 8)
    cache = CacheManager(needs, 4, 32, 2, torch.float32, "cpu")
    assert len(cache.groups) == 2 and isinstance(cache.view(1), tuple) and len(cache.view(1)) == 3
    assert cache.view(1)[1].k.dtype == torch.float32
    cache.append("a", 23)
    cache.commit("a")
    # 23 positions: pages of 4 for the window's tokens (older ones given back), 4 complete blocks of 5 -> 1 page
    assert len(cache.block_table("a", cache.view(1)[1].group)) == 1
    held = cache.block_table("a", cache.view(1)[0].group)
    assert len(held) == 6 and held[0] == -1 and held[-1] >= 0
    cache.append("a", 1)
    cache.commit("a")
    cache.check()
    cache.release("a")
    assert cache.free_pages()[0] == 32


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
    order and the attention folds keys from the start of each list, so cuts agree to rounding."""
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
def test_long_decoding_through_pages_that_are_given_back(tmp_path, backend):
    """200 tokens one by one after a short prompt, a second request joining half-way: the window
    passes over decoded tokens, pages behind it go back to the pool and are taken again (the trace
    runs twice in one engine, and claims more pages over that time than the pool has)."""
    doc, seed = DOCS["A"]
    tensors = helpers.make_folder(tmp_path, doc, seed, std=0.15)
    a = helpers.random_prompt(230, doc["vocab"], 5)
    b = helpers.random_prompt(110, doc["vocab"], 6)
    reference = {"a": reference_logits(doc, tensors, a), "b": reference_logits(doc, tensors, b)}
    steps = [([("a", a[:30], list(range(30)))], [])]
    for i in range(30, 230):
        entries = [("a", [a[i]], [0])]
        j = i - 130  # b: a prompt of 20 at a's position 130, then one token a step
        if j == 0:
            entries.insert(0, ("b", b[:20], list(range(20))))
        elif 0 < j <= 90:
            entries.append(("b", [b[19 + j]], [0]))
        steps.append((entries, [r for r, n in (("a", 229), ("b", 220)) if i == n]))
    for dtype in dtypes(backend):
        engine = helpers.make_engine(tmp_path, dtype, page_size=4, kv_cache_tokens=352, ctx=240, max_num_batched_tokens=64,
                                     **backend_args(backend))
        most = 0
        for step in steps[:150]:
            rows = helpers.run_steps(engine, [step])
            most = max(most, 88 - engine.cache.free_pages()[0])
        assert most <= 2 * 4 + 2  # two requests hold their windows (9 positions, blocks of 5), not their lengths
        engine.finish("a"), engine.finish("b")
        rows = helpers.run_steps(engine, steps)
        check_rows(replay.stack_rows(rows, "a", 230), reference["a"], dtype, f"long decoding {dtype}")
        check_rows(replay.stack_rows(rows, "b", 110), reference["b"], dtype, f"the request that joined {dtype}")
        assert engine.cache.free_pages()[0] == 88 and engine.cache.slots.free_slots == 4


DOC_WIDE = {
    "architecture": "Filulix", "vocab": 400, "width": 128, "streams": 2, "norm": {"eps": 1e-6},
    "embedding": {"scale": 4.0, "bigram": {"buckets": 211, "mul_prev": 29, "mul_cur": 3}},
    "layers": [
        parallel_layer(
            {"heads": 6, "kv_heads": 3, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": 200, "pool": 24}},
            {"heads": 2, "dim": 16, "vdim": 32, "decay": [0.97, 0.999], "rot": {"dims": 16, "base": 10000.0}},
            (0.8, 0.6), 160),
        wkv_layer(2, 64, 8, 160),
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}


@pytest.mark.gpu
def test_long_bfloat16_portions_take_the_tensor_memory_window(tmp_path):
    """Heads of 64 in bfloat16: a step with a long portion sends the window's tokens to the
    tensor-memory attention kernel and folds the pooled blocks in afterwards; shorter portions and
    decoded tokens take the general kernel.  Both against the plain implementation, whole, in
    portions on either side of the route's limits, and with a second request in the batch."""
    tensors = helpers.make_folder(tmp_path, DOC_WIDE, 9, std=0.08)
    a = helpers.random_prompt(700, DOC_WIDE["vocab"], 1)
    b = helpers.random_prompt(150, DOC_WIDE["vocab"], 2)
    reference = {"a": reference_logits(DOC_WIDE, tensors, a), "b": reference_logits(DOC_WIDE, tensors, b)}
    for dtype in ("bfloat16", "float32"):
        engine = helpers.make_engine(tmp_path, dtype, page_size=16, kv_cache_tokens=2048, ctx=1024, max_num_batched_tokens=1024)
        rows = helpers.run_steps(engine, helpers.whole("w", a))
        check_rows(replay.stack_rows(rows, "w", 700), reference["a"], dtype, f"one long portion {dtype}")
        rows = helpers.run_steps(engine, helpers.portions("p", a, [300, 100, 260, 1, 39]))
        check_rows(replay.stack_rows(rows, "p", 700), reference["a"], dtype, f"long and short portions {dtype}")
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
    doc, seed = DOCS["A"]
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
        self.builder = StepBuilder(self.cache, env.device, 512, slots)

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


WKV = PartSpec("wkv_time_mix", {
    "hidden_size": 40, "num_heads": 5, "head_dim": 12, "eps": 1e-5, "decay_rank": 6,
    "mu": {c: f"m.mu.{c}" for c in "rkvgw"}, "r_proj": "m.r", "k_proj": "m.k", "v_proj": "m.v", "g_proj": "m.g",
    "decay_down": "m.w1", "decay_up": "m.w2", "decay_bias": "m.w0", "bonus": "m.u", "out_norm": "m.norm", "out_proj": "m.o",
})


@pytest.mark.parametrize("backend", BACKENDS)
def test_wkv_mixer_alone_in_steps_and_batches(backend):
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        mixer = MIXERS.build(WKV, env)
        w = bind(mixer, env, 11)
        spec = {"heads": 5, "dim": 12}
        g = torch.Generator().manual_seed(1)
        a, b = torch.randn(37, 40, generator=g).to(dtype), torch.randn(9, 40, generator=g).to(dtype)
        want_a = plain.wkv_mixer({k.replace("m.", "l0.mix."): v for k, v in w.items()}, "l0", spec, a.double(), 1e-5)
        want_b = plain.wkv_mixer({k.replace("m.", "l0.mix."): v for k, v in w.items()}, "l0", spec, b.double(), 1e-5)
        feeder = Feeder(mixer, env)
        got_a, got_b = [], []
        out = feeder.step([("a", a[:20]), ("b", b[:1])])  # a portion beside a single token
        got_a.append(out["a"]); got_b.append(out["b"])
        out = feeder.step([("b", b[1:3]), ("a", a[20:22])])  # two tokens each, order swapped
        got_a.append(out["a"]); got_b.append(out["b"])
        out = feeder.step([("a", a[22:23])])
        got_a.append(out["a"])
        out = feeder.step([("a", a[23:]), ("b", b[3:])])
        got_a.append(out["a"]); got_b.append(out["b"])
        close(torch.cat(got_a), want_a, dtype, f"wkv a {dtype}", 4.0)
        close(torch.cat(got_b), want_b, dtype, f"wkv b {dtype}", 4.0)
        # a slot that is given back and taken again starts from zero
        feeder.cache.release("a")
        again = feeder.step([("c", a[:5])])["c"]
        close(again, want_a[:5], dtype, f"wkv in a slot used again {dtype}", 4.0)


def attention_spec(heads, kv_heads, dim, vdim, window, pool, scale):
    return PartSpec("pooled_window_attention", {
        "hidden_size": 32, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": dim, "v_head_dim": vdim,
        "scale": scale, "window": window, "pool": pool, "q_proj": "a.q", "k_proj": "a.k", "v_proj": "a.v", "out_proj": "a.o",
    })


def plain_attention_mixer(w, heads, kv_heads, dim, vdim, window, pool, scale, h, cache_dtype=None):
    T = h.shape[0]
    q = (h @ w["a.q"].T).reshape(T, heads, dim)
    k = (h @ w["a.k"].T).reshape(T, kv_heads, dim)
    v = (h @ w["a.v"].T).reshape(T, kv_heads, vdim)
    if cache_dtype is not None:
        q, k, v = (t.to(cache_dtype).double() for t in (q, k, v))
    return plain.pooled_window_attention(q, k, v, scale, window, pool).reshape(T, heads * vdim) @ w["a.o"].T


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("shape", [(4, 2, 8, 12, 7, 3), (3, 3, 20, 4, 5, 5), (2, 1, 16, 16, 1, 1), (2, 1, 6, 10, 4, 9)])
def test_pooled_window_attention_alone(backend, shape):
    heads, kv_heads, dim, vdim, window, pool = shape
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        mixer = MIXERS.build(attention_spec(heads, kv_heads, dim, vdim, window, pool, 0.4), env)
        w = bind(mixer, env, 21, 0.3)
        g = torch.Generator().manual_seed(2)
        a, b = torch.randn(41, 32, generator=g).to(dtype), torch.randn(13, 32, generator=g).to(dtype)
        rounded = None if dtype == torch.float32 else dtype
        want_a = plain_attention_mixer(w, heads, kv_heads, dim, vdim, window, pool, 0.4, a.double(), rounded)
        want_b = plain_attention_mixer(w, heads, kv_heads, dim, vdim, window, pool, 0.4, b.double(), rounded)
        feeder = Feeder(mixer, env)
        got_a, got_b = [], []
        for cut_a, cut_b in (((0, 11), (0, 1)), ((11, 13), (1, 2)), ((13, 14), (2, 9)), ((14, 41), (9, 13))):
            out = feeder.step([("a", a[cut_a[0] : cut_a[1]]), ("b", b[cut_b[0] : cut_b[1]])])
            got_a.append(out["a"]); got_b.append(out["b"])
        close(torch.cat(got_a), want_a, dtype, f"attention a {shape} {dtype}", 2.0)
        close(torch.cat(got_b), want_b, dtype, f"attention b {shape} {dtype}", 2.0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_a_planted_key_shows_at_every_edge_of_window_and_blocks(backend):
    """One key is made to stand out (its query direction scaled up), so that whether it is seen,
    seen through its block's mean, or not seen at all decides the output: the key sits far back
    among hundreds, at page borders, just inside and just outside the window, and in a block
    that is just behind the window or not yet; the query comes in a prompt and as a decoded token."""
    heads, kv_heads, dim, vdim, window, pool = 2, 1, 8, 8, 12, 5
    dtype = torch.float32
    env = build_env(backend, dtype)
    mixer = MIXERS.build(attention_spec(heads, kv_heads, dim, vdim, window, pool, 1.0), env)
    w = bind(mixer, env, 31, 0.3)
    T = 300
    g = torch.Generator().manual_seed(3)
    base = torch.randn(T, 32, generator=g) * 0.1
    # a direction that the key matrix maps to a large key along the query of the probe rows
    probe = torch.randn(32, generator=g)
    for planted in (0, 3, 4, 5, 150, 251, 252, 283, 284, 287, 288, 289, 299):
        h = base.clone()
        h[planted] = probe * 3.0
        h[T - 1] = probe * 3.0  # the last row asks for it
        want = plain_attention_mixer(w, heads, kv_heads, dim, vdim, window, pool, 1.0, h.double())
        for tail in (0, 40):  # the asking row inside a prompt's portion, or decoded after 40 single tokens
            feeder = Feeder(mixer, env, pages=128)
            got = [feeder.step([("a", h[: T - tail - 7])])["a"], feeder.step([("a", h[T - tail - 7 : T - tail])])["a"]]
            for t in range(T - tail, T):
                got.append(feeder.step([("a", h[t : t + 1])])["a"])
            close(torch.cat(got), want, dtype, f"planted at {planted}, {tail} decoded", 2.0)


RETENTION = PartSpec("retention", {
    "hidden_size": 24, "num_heads": 3, "head_dim": 10, "v_head_dim": 6, "decay": (0.5, 0.95, 1.0), "eps": 1e-6,
    "position": PartSpec("rope_half_split", {"theta": 50.0, "rotary_dim": 6}),
    "q_proj": "r.q", "k_proj": "r.k", "v_proj": "r.v", "g_proj": "r.g", "out_proj": "r.o",
})


@pytest.mark.parametrize("backend", BACKENDS)
def test_retention_alone_with_partial_rotation(backend):
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        mixer = MIXERS.build(RETENTION, env)
        w = bind(mixer, env, 41, 0.3)
        g = torch.Generator().manual_seed(4)
        a = torch.randn(50, 24, generator=g).to(dtype)
        h = a.double()
        T = 50
        rnd = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(dtype).double())
        q = rnd(h @ w["r.q"].T).reshape(T, 3, 10)
        k = rnd(h @ w["r.k"].T).reshape(T, 3, 10)
        v = rnd(h @ w["r.v"].T).reshape(T, 3, 6)
        gate = rnd(h @ w["r.g"].T)
        q = plain.rotate_half_split(q, list(range(T)), 6, 50.0)
        k = plain.rotate_half_split(k, list(range(T)), 6, 50.0) * 10 ** -0.5
        o = plain.rms_unit(plain.retention(q, k, v, (0.5, 0.95, 1.0)), 1e-6).reshape(T, 18) * plain.silu(gate)
        want = rnd(o) @ w["r.o"].T
        feeder = Feeder(mixer, env)
        got = [feeder.step([("a", a[:17])])["a"], feeder.step([("a", a[17:19])])["a"]]
        got += [feeder.step([("a", a[t : t + 1])])["a"] for t in range(19, 30)]
        got.append(feeder.step([("a", a[30:])])["a"])
        close(torch.cat(got), want, dtype, f"retention {dtype}", 3.0)


@pytest.mark.parametrize("backend", BACKENDS)
def test_hashed_pair_embedding_and_its_state(backend):
    from shiso_llm_b200.parts import EMBEDDINGS

    env = build_env(backend, torch.float32)
    spec = PartSpec("hashed_pair_embedding", {"tensor": "e", "pair_tensor": "p", "vocab_size": 50, "hidden_size": 16,
                                              "scale": 3.0, "buckets": 7, "mul_prev": 5, "mul_cur": 11})
    emb = EMBEDDINGS.build(spec, env)
    w = bind(emb, env, 51, 1.0)
    cache = CacheManager([emb.cache_spec()], 4, 8, 2, torch.float32, env.device)
    builder = StepBuilder(cache, env.device, 64, 2)
    toks = {"a": [3, 49, 0, 7, 7, 12, 30], "b": [9, 9, 9]}
    doc = {"embedding": {"scale": 3.0, "bigram": {"buckets": 7, "mul_prev": 5, "mul_cur": 11}}}
    want = {r: plain.embedding(doc, {"embed": w["e"], "bigram": w["p"]}, t) for r, t in toks.items()}
    got = {"a": [], "b": []}
    for parts in ([("a", 0, 3), ("b", 0, 1)], [("b", 1, 3), ("a", 3, 4)], [("a", 4, 7)]):
        entries = [StepEntry(r, toks[r][lo:hi], []) for r, lo, hi in parts]
        starts = [cache.append(r, hi - lo) for r, lo, hi in parts]
        rows = emb.forward(builder.build(entries, starts), cache.view(0)).double().cpu()
        at = 0
        for r, lo, hi in parts:
            got[r].append(rows[at : at + hi - lo])
            at += hi - lo
            cache.commit(r)
    for r in toks:
        close(torch.cat(got[r]), want[r], torch.float32, f"embedding of {r}")


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("copies", [1, 2, 5])
def test_stream_copies_read_write_and_sum(backend, copies):
    for dtype in mixer_dtypes(backend):
        env = build_env(backend, dtype)
        ops = env.ops
        g = torch.Generator().manual_seed(6)
        T, H = 7, 72
        x = torch.randn(T, H, generator=g)
        y1, y2 = torch.randn(T, H, generator=g).to(dtype), torch.randn(T, H, generator=g).to(dtype)
        read = [torch.randn(copies, generator=g) for _ in range(2)]
        write = [torch.randn(copies, generator=g) for _ in range(2)]
        mix = [torch.randn(copies, copies, generator=g) for _ in range(2)]
        weight = torch.randn(H, generator=g)
        dev = lambda t: t.to(env.device)  # noqa: E731
        lanes = x.double()[None].repeat(copies, 1, 1)
        u = torch.einsum("s,std->td", read[0].double(), lanes)
        want_first = plain.rms_unit(u, 1e-5) * weight.double()
        lanes = torch.einsum("sr,std->rtd", mix[0].double(), lanes) + write[0].double()[:, None, None] * y1.double()[None]
        u = torch.einsum("s,std->td", read[1].double(), lanes)
        want_second = plain.rms_unit(u, 1e-5) * weight.double()
        lanes = torch.einsum("sr,std->rtd", mix[1].double(), lanes) + write[1].double()[:, None, None] * y2.double()[None]
        none, first = ops.hyper_mix_read(dev(x), None, None, None, copies, dev(read[0]), dev(weight), 1e-5, dtype)
        assert none is None
        held, second = ops.hyper_mix_read(dev(x), dev(y1), dev(mix[0]), dev(write[0]), copies, dev(read[1]), dev(weight), 1e-5, dtype)
        total = ops.hyper_mix_sum(held, dev(y2), dev(mix[1]), dev(write[1]))
        close(first.double().cpu(), want_first, dtype, "first read")
        close(second.double().cpu(), want_second, dtype, "write and read", 4.0)
        close(total.double().cpu(), lanes.sum(0), torch.float32, "write and sum", 4.0)
