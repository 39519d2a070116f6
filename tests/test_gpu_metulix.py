"""The Metulix design in the engine against the plain implementation of the tests: every
mechanism alone, whole prompts against decoding token by token, portions down to two tokens,
mixed batches with pages and state slots that are used again, window edges and kept first
tokens in prompts and in decoding, long decoding, and greedy generation through the engine."""

import numpy as np
import pytest
import torch

import helpers
import metulix_models as mm
import plain_metulix as plain

pytestmark = pytest.mark.gpu

F32_BOUND = 2e-4          # largest |engine - plain| of a row, relative to max(1, largest |plain|)
BF16_BOUND = 6e-2
# float32 runs the sharpened weights (a key too many or too few shows); bfloat16 runs the plain
# random weights, whose rounding error stays a few percent of the logits
SHARPEN = {"float32": True, "bfloat16": False}


_folders = {}
_plain = {}


def folder_of(tmp_path_factory, name, **options):
    key = (name, tuple(sorted(options.items())))
    if key not in _folders:
        _folders[key] = mm.write_model(tmp_path_factory.mktemp(f"metulix_{name}"), name, **options)
    return _folders[key]


def plain_rows(folder, ids):
    key = (str(folder), tuple(ids))
    if key not in _plain:
        _plain[key] = plain.logits_of(folder, ids).numpy()
    return _plain[key]


def runner_for(folder, dtype, num_pages, max_requests=4, page_size=16, **options):
    from from_scratch_inference_engine_b200 import LoadedModel, ModelRunner
    model = LoadedModel.from_pretrained(folder, dtype=dtype, max_positions=num_pages * page_size)
    return ModelRunner(model.model, model.runtime, page_size=page_size, num_pages=num_pages,
                       max_requests=max_requests, max_step_tokens=num_pages * page_size, **options)


def assert_rows(rows, requests, folder, bound):
    """Every row within `bound` of the plain logits.  bfloat16 rounds every product's result, and
    a norm on each sublayer's output passes the relative error of a small output on at full
    size: there one row in ten may lie beyond the bound, none beyond three times it."""
    assert rows
    beyond = 0
    for (key, pos), row in sorted(rows.items()):
        want = plain_rows(folder, requests[key.split("~")[0]])[pos]
        base = max(1.0, float(np.abs(want).max()))
        diff = float(np.abs(row.astype(np.float64) - want).max())
        limit = bound * base * (3.0 if bound == BF16_BOUND else 1.0)
        assert diff <= limit, f"request {key} position {pos}: off by {diff:.3e} (bound {limit:.3e})"
        beyond += diff > bound * base
    assert beyond <= 0.1 * len(rows), f"{beyond} of {len(rows)} rows beyond the bound"


def vocab_of(name):
    return mm.CONFIGS[name]["vocab"]


# ----------------------------------------------------------------- mechanisms, kernel by kernel
def test_layer_norm_kernels_against_the_formula():
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    for width in (36, 256, 1000):
        x = torch.randn(7, width, generator=g) * 3 + 1.5
        gain = torch.randn(width, generator=g)
        want = plain.layer_norm(x.double(), gain.double(), 1e-5)
        rows = torch.tensor([5, 0, 3], dtype=torch.int32)
        got = ops.layernorm_rows(x.cuda(), gain.cuda(), 1e-5, torch.empty(3, width, device="cuda"),
                                 rows=rows.cuda())
        assert (got.cpu().double() - want[rows.long()]).abs().max() < 1e-5
        base = torch.randn(7, width, generator=g)
        residual = base.clone().cuda()
        copy = torch.empty(7, width, device="cuda")
        ops.add_layernorm(residual, x.cuda(), gain.cuda(), 1e-5, copy)
        assert (residual.cpu().double() - (base.double() + want)).abs().max() < 1e-5
        assert torch.equal(copy, residual)
        delta16 = x.to(torch.bfloat16)
        residual = base.clone().cuda()
        copy16 = torch.empty(7, width, device="cuda", dtype=torch.bfloat16)
        ops.add_layernorm(residual, delta16.cuda(), gain.cuda(), 1e-5, copy16)
        want16 = base.double() + plain.layer_norm(delta16.double(), gain.double(), 1e-5)
        assert (residual.cpu().double() - want16).abs().max() < 1e-5       # the sum stays 32-bit
        assert torch.equal(copy16, residual.to(torch.bfloat16))


@pytest.mark.parametrize("heads,dim,vdim", [(3, 10, 24), (1, 64, 40), (2, 130, 33)])
def test_lightning_scan_carries_state_between_calls(heads, dim, vdim):
    """Two requests of unequal length in one call, then more tokens of both in a second call
    (one of them a single token): the state left in the slots carries the sum on."""
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(heads * 100 + dim)
    lengths = {"a": (9, 1), "b": (21, 6)}
    decay = torch.tensor([1.0, 0.5, 0.97][:heads])
    width = 2 * heads * dim + heads * vdim
    proj = {k: torch.randn(sum(n), width, generator=g) for k, n in lengths.items()}
    state = torch.full((3, heads, dim, vdim), 7.0, device="cuda")
    state[0].zero_()
    state[2].zero_()
    slots = torch.tensor([2, 0], dtype=torch.int32, device="cuda")
    outs = {k: [] for k in lengths}
    for call in range(2):
        parts = [proj[k][sum(lengths[k][:call]):sum(lengths[k][:call + 1])] for k in ("a", "b")]
        batch = torch.cat(parts).cuda()
        batch = ops.silu_rows(batch, width, torch.empty_like(batch))
        qlen = torch.tensor([len(p) for p in parts], dtype=torch.int32)
        qstart = torch.tensor([0, len(parts[0])], dtype=torch.int32)
        out = torch.empty(batch.shape[0], heads * vdim, device="cuda")
        ops.lightning_scan(batch, 0, heads * dim, 2 * heads * dim, qstart.cuda(), qlen.cuda(), slots,
                           2, state, decay.cuda(), out, heads, dim, vdim)
        outs["a"].append(out[:len(parts[0])].cpu())
        outs["b"].append(out[len(parts[0]):].cpu())
    assert float(state[1].min()) == 7.0                      # a slot nobody named is untouched
    for key, slot in (("a", 2), ("b", 0)):
        p = proj[key].double()
        T = p.shape[0]
        q = plain.silu(p[:, :heads * dim]).view(T, heads, dim)
        k = plain.silu(p[:, heads * dim:2 * heads * dim]).view(T, heads, dim)
        v = plain.silu(p[:, 2 * heads * dim:]).view(T, heads, vdim)
        want, final = plain.lightning_recurrence(q, k, v, decay.tolist())
        got = torch.cat(outs[key]).double().view(T, heads, vdim)
        scale = max(1.0, float(want.abs().max()))
        assert (got - want).abs().max() < 1e-5 * scale
        assert (state[slot].cpu().double() - final).abs().max() < 1e-5 * max(1.0, float(final.abs().max()))


def test_cache_keeps_the_pages_of_kept_first_tokens():
    """A windowed cache entry gives back the pages that no later query can see, except those
    of the kept first tokens; a reader with a wider window widens what the entry keeps."""
    from from_scratch_inference_engine_b200.cache.manager import CacheManager, CacheNeed
    need = CacheNeed(2, 8, window=10, keep_first=5, value_dim=12)
    assert need.v_dim == 12 and CacheNeed(2, 8).v_dim == 8
    cache = CacheManager([need], page_size=4, num_pages=12, num_slots=2)
    handle = cache.open("r")
    for _ in range(10):
        cache.reserve(handle, 4)
        cache.commit(handle, 4)
    table = handle.tables[0]
    assert table[0] >= 0 and table[1] >= 0                   # tokens 0..4 live in pages 0 and 1
    assert all(page < 0 for page in table[2:7]) and all(page >= 0 for page in table[7:])
    cache.check()
    wider = need.covering(CacheNeed(2, 8, window=30, keep_first=2, value_dim=12))
    assert (wider.window, wider.keep_first) == (30, 5)
    assert need.covering(CacheNeed(2, 8, window=0, value_dim=12)).window == 0
    with pytest.raises(ValueError):
        need.covering(CacheNeed(2, 8, window=10))


# ------------------------------------------------------------------- each mixer alone, in a model
@pytest.mark.parametrize("name", ["attention", "lightning", "odd"])
def test_one_mixer_whole_prompt_and_token_by_token(tmp_path_factory, name):
    """The prompt in one step against the same tokens one by one: the first tokens of a sequence
    (zeros before the convolution's start, an empty state), every window edge, the kept first
    tokens, page borders - as a prompt's rows and as decoded tokens."""
    folder = folder_of(tmp_path_factory, name)
    requests = {"p": helpers.random_ids(vocab_of(name), 70, 11)}
    runner = runner_for(folder, "float32", num_pages=8)
    rows = helpers.run_trace_in_process(runner, helpers.trace_whole(requests))
    assert len(rows) == 70
    assert_rows(rows, requests, folder, F32_BOUND)
    rows = helpers.run_trace_in_process(runner, helpers.trace_tail_by_one(requests, tail=69))
    assert len(rows) == 70
    assert_rows(rows, requests, folder, F32_BOUND)


@pytest.mark.parametrize("name", ["lightning", "hybrid"])
def test_long_prompt_sums_chunk_by_chunk(tmp_path_factory, name):
    """A prompt long enough that the linear attention runs its chunks side by side (sums per
    chunk, chained, then the outputs), whole and cut in two inside a chunk, beside a short
    request in the same step; then decoding goes on from the state the chunks left."""
    folder = folder_of(tmp_path_factory, name)
    requests = {"long": helpers.random_ids(vocab_of(name), 331, 3),
                "short": helpers.random_ids(vocab_of(name), 12, 4)}
    runner = runner_for(folder, "float32", num_pages=48)
    steps = [{"step": 0, "end": ["short"], "entries": [
                  {"id": "long", "tokens": requests["long"][:203], "want": [0, 63, 64, 127, 128, 202]},
                  {"id": "short", "tokens": requests["short"], "want": [11]}]},
             {"step": 1, "end": [], "entries": [
                  {"id": "long", "tokens": requests["long"][203:329], "want": [0, 60, 125]}]},
             {"step": 2, "end": [], "entries": [{"id": "long", "tokens": [requests["long"][329]], "want": [0]}]},
             {"step": 3, "end": ["long"], "entries": [{"id": "long", "tokens": [requests["long"][330]], "want": [0]}]}]
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) == 12
    assert_rows(rows, requests, folder, F32_BOUND)


def test_sizes_that_fit_no_vector_in_bfloat16(tmp_path_factory):
    """Width 36, feed-forward 50, vocabulary 61, head sizes 6 and 10: no row starts on 16 bytes.
    The bfloat16 products and kernels take their plain forms; prompt, portions and decoding."""
    folder = folder_of(tmp_path_factory, "odd", sharpen=False)
    requests = {"a": helpers.random_ids(vocab_of("odd"), 45, 6), "b": helpers.random_ids(vocab_of("odd"), 19, 7)}
    runner = runner_for(folder, "bfloat16", num_pages=8)
    for steps in (helpers.trace_whole(requests), helpers.trace_mixed(requests, seed=1, max_live=2)):
        rows = helpers.run_trace_in_process(runner, steps)
        assert len(rows) == 64
        assert_rows(rows, requests, folder, BF16_BOUND)


def test_window_edge_shows_in_the_logits(tmp_path_factory):
    """The test model's softmax is sharp enough that dropping the key at the window's far edge,
    or admitting the one beyond it, or dropping the kept first tokens, moves the logits far
    beyond the bound that the engine is held to: the comparisons above can tell."""
    folder = folder_of(tmp_path_factory, "attention")
    config, weights = plain.load(folder)
    ids = helpers.random_ids(vocab_of("attention"), 60, 11)
    right = plain.forward(config, weights, ids)
    scale = max(1.0, float(right.abs().max()))
    for size, keep in ((10, 3), (12, 3), (11, 0)):
        config["layers"][0]["mixer"]["mask"] = {"size": size, "keep_first": keep}
        wrong = plain.forward(config, weights, ids)
        assert float((wrong - right).abs().max()) > 50 * F32_BOUND * scale


# ---------------------------------------------------------------------------- the whole design
@pytest.mark.parametrize("dtype,bound", [("float32", F32_BOUND), ("bfloat16", BF16_BOUND)])
def test_hybrid_portions_of_every_size(tmp_path_factory, dtype, bound):
    folder = folder_of(tmp_path_factory, "hybrid", sharpen=SHARPEN[dtype])
    requests = {"a": helpers.random_ids(vocab_of("hybrid"), 90, 1),
                "b": helpers.random_ids(vocab_of("hybrid"), 37, 2)}
    runner = runner_for(folder, dtype, num_pages=8)
    steps = helpers.trace_portions(requests, seed=3)
    assert min(len(e["tokens"]) for s in steps for e in s["entries"]) <= 2
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) == 127
    assert_rows(rows, requests, folder, bound)


@pytest.mark.parametrize("dtype,bound", [("float32", F32_BOUND), ("bfloat16", BF16_BOUND)])
def test_hybrid_mixed_batches_reuse_pages_and_slots(tmp_path_factory, dtype, bound):
    """Six unequal requests through two state slots and a pool that holds little more than two of
    them: portions of one beside single tokens of another, requests that sit a step out, one
    that is released in the middle and fed again from its first token - every request's rows
    equal what it gives alone."""
    folder = folder_of(tmp_path_factory, "hybrid", sharpen=SHARPEN[dtype])
    lengths = {"a": 75, "b": 9, "c": 41, "d": 1, "e": 58, "f": 26}
    requests = {k: helpers.random_ids(vocab_of("hybrid"), n, i + 20)
                for i, (k, n) in enumerate(lengths.items())}
    steps, names = helpers.trace_mixed_with_recompute(requests, seed=5, max_live=2)
    need = helpers.live_tokens_needed(steps, round_to=16)
    runner = runner_for(folder, dtype, num_pages=need // 16, max_requests=2)
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) >= sum(lengths.values())
    assert_rows(rows, names, folder, bound)
    assert runner.cache.slots.num_free == 2
    assert all(free == need // 16 for free in runner.cache.free_pages())


def test_tensor_core_attention_against_the_32_bit_form_and_plain(tmp_path_factory):
    """bfloat16 prompt portions at head size 64 run the tensor-core form (mixing on the output
    side); the same requests with that form switched off run the 32-bit form.  Both lie within
    the bfloat16 bound of the plain logits and close to one another; portions start and end
    inside tiles of 16 tokens, windows end inside tiles, single tokens ride along."""
    folder = folder_of(tmp_path_factory, "wide", sharpen=False)
    lengths = {"a": 133, "b": 47, "c": 90}
    requests = {k: helpers.random_ids(vocab_of("wide"), n, i + 40) for i, (k, n) in enumerate(lengths.items())}
    steps = helpers.trace_mixed(requests, seed=8, max_live=3) + [
        dict(s, step=1000 + s["step"]) for s in helpers.trace_whole({k + "~w": v for k, v in requests.items()})]
    names = dict(requests)
    names.update({k + "~w": v for k, v in requests.items()})
    both = []
    for tensor_cores in (True, False):
        runner = runner_for(folder, "bfloat16", num_pages=40, max_requests=3)
        mixers = [block.mixer for block in runner.model.blocks if hasattr(block.mixer, "tensor_cores")]
        assert len(mixers) == 2 and all(m.tensor_cores for m in mixers)
        for mixer in mixers:
            mixer.tensor_cores = tensor_cores
        rows = helpers.run_trace_in_process(runner, steps)
        assert_rows(rows, names, folder, BF16_BOUND)
        both.append(rows)
    for key, row in both[0].items():
        other = both[1][key]
        assert float(np.abs(row - other).max()) <= 3e-2 * max(1.0, float(np.abs(other).max())), key


def test_hybrid_long_decoding_through_graphs_and_without(tmp_path_factory):
    """A short prompt, then 150 tokens one by one: the window and the kept first tokens pass
    over decoded tokens, pages are given back on the way, and the decode steps replay captured
    graphs; the same without graphs gives the same rows."""
    folder = folder_of(tmp_path_factory, "hybrid")
    requests = {"long": helpers.random_ids(vocab_of("hybrid"), 157, 9)}
    steps = helpers.trace_tail_by_one(requests, tail=150)
    both = []
    for graphs in (True, False):
        runner = runner_for(folder, "float32", num_pages=12, cuda_graphs=graphs)
        assert runner.cuda_graphs == graphs
        rows = helpers.run_trace_in_process(runner, steps)
        assert_rows(rows, requests, folder, F32_BOUND)
        both.append(rows)
    for key in both[0]:
        assert np.array_equal(both[0][key], both[1][key])


def test_decode_batch_with_padding_leaves_other_slots_alone(tmp_path_factory):
    """Three requests decode together in a captured batch of four: the padding entry must not
    touch the state of slot 0, which a live request holds."""
    folder = folder_of(tmp_path_factory, "hybrid")
    requests = {k: helpers.random_ids(vocab_of("hybrid"), n, s)
                for k, n, s in (("a", 30, 1), ("b", 22, 2), ("c", 26, 3))}
    runner = runner_for(folder, "float32", num_pages=12)
    steps = [{"step": 0, "end": [], "entries": [
        {"id": k, "tokens": ids[:12], "want": [11]} for k, ids in requests.items()]}]
    for t in range(12, 22):
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": k, "tokens": [ids[t]], "want": [0]} for k, ids in requests.items()]})
    steps[-1]["end"] = list(requests)
    rows = helpers.run_trace_in_process(runner, steps)
    assert runner._graphs
    assert_rows(rows, requests, folder, F32_BOUND)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tmp_path_factory, dtype):
    """Requests of unequal length through `Engine` and its scheduler with a small token budget
    (prompts go in portions) and two slots: every generated token is the plain implementation's
    choice; where the plain logits are a near tie the engine may pick either."""
    from from_scratch_inference_engine_b200 import Engine, LoadedModel, SamplingParams
    folder = folder_of(tmp_path_factory, "hybrid", sharpen=SHARPEN[dtype])
    model = LoadedModel.from_pretrained(folder, dtype=dtype, max_positions=256)
    engine = Engine(model, block_size=16, num_blocks=16, max_batch=2, max_step_tokens=24)
    prompts = [helpers.random_ids(vocab_of("hybrid"), n, s) for n, s in ((45, 1), (7, 2), (30, 3))]
    ids = [engine.add_request(p, SamplingParams(temperature=0.0), 8) for p in prompts]
    engine.run_until_done()
    config, weights = plain.load(folder)
    slack = 1e-3 if dtype == "float32" else 0.15
    for rid, prompt in zip(ids, prompts):
        seq = list(prompt)
        assert len(engine.output(rid)) == 8
        for token in engine.output(rid):
            logits = plain.forward(config, weights, seq)[-1]
            assert float(logits.max() - logits[token]) <= slack * max(1.0, float(logits.abs().max()))
            seq.append(token)


def test_llm_entry_point_reads_the_design_by_its_name(tmp_path_factory):
    from from_scratch_inference_engine_b200 import LLM, GenerationConfig, load_config
    folder = folder_of(tmp_path_factory, "odd")
    assert type(load_config(folder)).__name__ == "MetulixConfig"
    llm = LLM(folder, block_size=16, num_blocks=8, max_batch=2, dtype="float32", eos_id=-1)
    prompt = helpers.random_ids(vocab_of("odd"), 19, 4)
    got = llm.generate_ids(prompt, GenerationConfig(max_tokens=5))
    config, weights = plain.load(folder)
    seq = list(prompt)
    for token in got:
        logits = plain.forward(config, weights, seq)[-1]
        assert float(logits.max() - logits[token]) <= 1e-3 * max(1.0, float(logits.abs().max()))
        seq.append(token)
