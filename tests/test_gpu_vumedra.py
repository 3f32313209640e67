"""The Vumedra design in the engine against its plain restatement: every mechanism alone in a model of one layer,
whole prompts, prompts followed by single tokens, portions of many sizes down to two tokens, unequal batches, caches so
small that slots, pages and state rows are used again, long decoding, greedy generation through the entry point and
the command line, and the replay program."""
import functools
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_vumedra as plain
from gpu_util import Recorder, run_steps, steps_batches, steps_tail, steps_whole
from test_gpu_zusepel import steps_portions
from tiny import repo_root
from vumedra_cases import case, one_layer, random_weights

from esp_b200.engine import Engine, StepEntry
from esp_b200.weights import write_safetensors

pytestmark = pytest.mark.gpu

# root mean square of (engine - plain) over a row of logits, mean taken off, over the root mean square of the
# request's plain logits.  float32: the order of sums differs, and the matrix memory divides by max(|n . q|, exp(-m)),
# a sum of 32-bit terms that may partly cancel, which magnifies their rounding: the plain restatement itself, run in
# 32-bit, is off by up to 2.5e-5 on these models (on 303 tokens through the second configuration; 4e-6 elsewhere).
# bfloat16: matrix products take rounded activations and the cache holds rounded keys and values; norms, gates and
# states stay 32-bit.
BOUND = {"float32": 5e-5, "bfloat16": 4e-2}

ALONE = {
    "attention": {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 32, "scale": 0.25,
                                                 "q_temp": {"coef": 0.6, "every": 5}}, "mlp": None},
    "attention_plain_kernel": {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 12, "vdim": 20, "scale": 0.4},
                               "mlp": None},
    "attention_equal_sizes": {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.11,
                                                             "q_temp": {"coef": 0.3, "every": 64}}, "mlp": None},
    "mlstm": {"type": "mlstm", "mixer": {"heads": 2, "dim": 24, "vdim": 40, "gate_cap": 10.0}, "mlp": None},
    "rglru": {"type": "rglru", "mixer": {"width": 48, "blocks": 2, "conv": 3}, "mlp": None},
    "dense": {"type": "rglru", "mixer": {"width": 16, "blocks": 1, "conv": 2}, "mlp": {"kind": "dense", "ff": 72}},
    "moe": {"type": "rglru", "mixer": {"width": 16, "blocks": 1, "conv": 2},
            "mlp": {"kind": "moe", "router": {"experts": 7, "top": 2}, "expert": {"ff": 24}, "shared": {"ff": 40}}},
    # a width of 128 and experts of 32: long steps take the router's tensor-core logits and the grouped TMA + tcgen05 products
    "moe_wide": {"type": "rglru", "mixer": {"width": 32, "blocks": 2, "conv": 2}, "width": 128,
                 "mlp": {"kind": "moe", "router": {"experts": 4, "top": 2}, "expert": {"ff": 32}, "shared": {"ff": 16}}},
}


@functools.lru_cache(maxsize=None)
def model(name, seed=7):
    if name in ALONE:
        layer = dict(ALONE[name])
        raw = one_layer(layer, width=layer.pop("width", 64))
    else:
        raw = case(name)
    stored = random_weights(raw, seed)
    return raw, stored, {k: v.double() for k, v in stored.items()}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            raw, stored, _ = model(name)
            d = tmp_path_factory.mktemp(f"vumedra_{name}")
            (d / "config.json").write_text(json.dumps(raw))
            write_safetensors(d / "model.safetensors", stored)
            made[name] = d
        return made[name]
    return get


_engines = {}


def engine_for(folder, dtype, max_tokens=2048, record=True, **kw):
    """``record``: the engine notes its expert choices, which the plain restatement then uses (a score within
    rounding of another may fall either way); such an engine replays no captured graphs."""
    key = (str(folder), dtype, max_tokens, record, tuple(sorted(kw.items())))
    if key not in _engines:
        _engines[key] = Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)
        _engines[key].rt.record_routing = record
    return _engines[key]


class Choices(Recorder):
    """Logits by (request, position) and the engine's expert choices by (request, layer, position)."""

    def take(self, entries, ids_of, logits, aux):
        routing = aux.pop("routing", [])
        super().take(entries, ids_of, logits, aux)
        for prefix, row0, ids, _w, _p in routing:
            layer = int(re.match(r"l(\d+)\.", prefix).group(1))
            ids = ids.cpu().numpy()
            start = 0
            for rid, first, n, _want in entries:
                for r in range(max(start, row0), min(start + n, row0 + ids.shape[0])):
                    self.routing.setdefault(rid, {}).setdefault(layer, {})[first + (r - start)] = ids[r - row0]
                start += n

    def chosen(self, rid, length):
        return {layer: torch.as_tensor(np.stack([by_pos[p] for p in range(length)]))
                for layer, by_pos in self.routing.get(rid, {}).items()}


def requests_for(name, lengths, seed=3):
    rng = np.random.default_rng(seed)
    vocab = model(name)[0]["vocab"]
    return {f"r{i}": [int(t) for t in rng.integers(0, vocab, n)] for i, n in enumerate(lengths)}


def check(name, dtype, requests, rec, what, positions=None):
    raw, _, w = model(name)
    for rid, toks in requests.items():
        chosen = rec.chosen(rid, len(toks)) if isinstance(rec, Choices) else {}
        ref = plain.forward(raw, w, toks, choices=chosen or None).numpy()
        if chosen and dtype == "float32":
            # in 32-bit the engine's choices are the plain ones (no score of these tests is that close to another)
            own = plain.forward(raw, w, toks).numpy()
            assert np.abs(own - ref).max() == 0, f"{what}: an expert choice of the engine differs from the plain one"
        at = list(range(len(toks))) if positions is None else list(positions[rid])
        got = rec.logits_of(rid, at)
        d = got - ref[at]
        d = d - d.mean(1, keepdims=True)
        err = np.sqrt((d ** 2).mean(1)) / np.sqrt((ref ** 2).mean())
        worst = int(np.argmax(err))
        assert err[worst] <= BOUND[dtype], (f"{what}, case {name}, {dtype}, request {rid} ({len(toks)} tokens): position "
                                            f"{at[worst]} is off by {err[worst]:.3e} (bound {BOUND[dtype]:.0e}); first "
                                            f"position over the bound: {at[int(np.argmax(err > BOUND[dtype]))]}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALONE))
def test_each_mechanism_alone(folders, name, dtype):
    """A model of one layer: whole prompts (the first token, a page's border), then prompt + single tokens."""
    reqs = requests_for(name, (1, 2, 64, 65, 150))
    eng = engine_for(folders(name), dtype)
    rec = Choices(model(name)[0]["vocab"])
    run_steps(eng, steps_whole(reqs), rec)
    check(name, dtype, reqs, rec, "one layer, whole prompts")
    rec = Choices(model(name)[0]["vocab"])
    run_steps(eng, steps_tail(reqs, tail=70), rec)
    check(name, dtype, reqs, rec, "one layer, prompt then single tokens")


LENGTHS = {"A": (1, 9, 83, 150), "B": (2, 40, 77, 131)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompts(folders, name, dtype):
    reqs = requests_for(name, LENGTHS[name])
    eng = engine_for(folders(name), dtype)
    rec = Choices(model(name)[0]["vocab"])
    run_steps(eng, steps_whole(reqs), rec)
    check(name, dtype, reqs, rec, "whole prompts")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_prefill_then_token_by_token(folders, name, dtype):
    """The last 80 tokens one by one: they pass page borders at 64 and 128 and many steps of the queries' temperature;
    the first requests are decoded from their second token on."""
    reqs = requests_for(name, LENGTHS[name])
    eng = engine_for(folders(name), dtype)
    rec = Choices(model(name)[0]["vocab"])
    run_steps(eng, steps_tail(reqs, tail=80), rec)
    check(name, dtype, reqs, rec, "prompt, then single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_of_many_sizes(folders, name, dtype):
    """Portions of two tokens are shorter than the convolution's reach (four taps): its state is shifted, not replaced."""
    reqs = requests_for(name, LENGTHS[name][1:], seed=5)
    eng = engine_for(folders(name), dtype)
    rec = Choices(model(name)[0]["vocab"])
    run_steps(eng, steps_portions(reqs, [2, 31, 3, 64, 17, 2, 2, 1, 2]), rec)
    check(name, dtype, reqs, rec, "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_in_a_cache_that_is_used_again(folders, name, dtype):
    """Two batches, one after the other, in a cache that holds one of them: every slot, page and state row (the
    recurrences', the convolution's, the token before) of the second batch was used by the first."""
    lengths = (70, 5, 140, 33, 129, 64, 2, 100)
    reqs = requests_for(name, lengths, seed=9)
    ids = list(reqs)
    batches = [ids[:4], ids[4:]]
    prompt = {rid: min(len(reqs[rid]), max(1, len(reqs[rid]) - 40 + 7 * i)) for i, rid in enumerate(ids)}
    eng = engine_for(folders(name), dtype, max_tokens=7 * 64, max_slots=4)
    rec = Choices(model(name)[0]["vocab"])
    run_steps(eng, steps_batches(reqs, batches, prompt), rec)
    check(name, dtype, reqs, rec, "unequal batches")
    assert eng.cache.book.slots.available == 4
    assert all(g.pool.available == g.pool.n for g in eng.cache.book.groups)


@pytest.mark.parametrize("name", ["A", "B"])
def test_cuttings_agree_bit_for_bit_in_float32(folders, name):
    """No sum's order depends on how a sequence is cut or what it is batched with; decode steps replay captured graphs."""
    reqs = requests_for(name, (3, 90, 150), seed=13)
    eng = engine_for(folders(name), "float32", record=False)
    outs = []
    ids = list(reqs)
    for steps in (steps_whole(reqs), steps_tail(reqs, tail=40), steps_portions(reqs, [2, 5, 64]),
                  steps_batches(reqs, [ids], {rid: max(1, len(t) - 30) for rid, t in reqs.items()})):
        rec = Recorder(model(name)[0]["vocab"])
        run_steps(eng, steps, rec)
        outs.append(rec)
    assert eng.graph_replays > 0
    for rid, toks in reqs.items():
        at = list(range(len(toks)))
        first = outs[0].logits_of(rid, at)
        for other in outs[1:]:
            assert np.array_equal(first, other.logits_of(rid, at))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_decode_steps_in_other_slots(folders, dtype):
    """Decode steps replayed from captured graphs, for sequences in other slots and pages than the ones the graph was
    captured with: slots, pages and state rows come from the step's device lists."""
    name = "A"
    reqs = requests_for(name, (40, 41, 100, 70), seed=23)
    eng = engine_for(folders(name), dtype, record=False)
    replays = eng.graph_replays
    rec = Recorder(model(name)[0]["vocab"])
    run_steps(eng, steps_tail(reqs, tail=30), rec)
    assert eng.graph_replays > replays
    if dtype == "float32" or all(l["mlp"] is None or l["mlp"]["kind"] == "dense" for l in model(name)[0]["layers"]):
        check(name, dtype, reqs, rec, "captured decode steps")
    else:
        # without the engine's expert choices a bfloat16 row may sit on the other side of a near tie: hold it against
        # the recording engine instead
        other = Choices(model(name)[0]["vocab"])
        run_steps(engine_for(folders(name), dtype), steps_tail(reqs, tail=30), other)
        for rid, toks in reqs.items():
            at = list(range(len(toks)))
            assert np.array_equal(rec.logits_of(rid, at), other.logits_of(rid, at))


def test_long_decoding(folders):
    """300 single tokens after a prompt of 3: states carried over hundreds of steps, five pages."""
    name = "A"
    reqs = requests_for(name, (303,), seed=21)
    for dtype in ("float32", "bfloat16"):
        eng = engine_for(folders(name), dtype, max_tokens=5 * 64)
        rec = Choices(model(name)[0]["vocab"])
        run_steps(eng, steps_tail(reqs, tail=300), rec)
        check(name, dtype, reqs, rec, "long decoding")


def test_residual_stream_behind_every_layer(folders):
    name = "A"
    raw, _, w = model(name)
    toks = requests_for(name, (45,), seed=2)["r0"]
    layers = []
    plain.forward(raw, w, toks, trace=layers)
    eng = engine_for(folders(name), "float32", record=False)
    slot = eng.open()
    aux = {"residual_trace": []}
    eng.step([StepEntry(slot, toks, [0])], aux)
    eng.close(slot)
    assert len(aux["residual_trace"]) == len(layers)
    for i, (got, want) in enumerate(zip(aux["residual_trace"], layers)):
        err = float((got.cpu().double() - want).abs().max() / want.abs().max())
        assert err < 1e-5, f"layer {i}: {err:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folders, dtype):
    from esp_b200.provider import DecoderProvider, GenerationRequest
    name = "B"
    raw, _, w = model(name)
    prompts = list(requests_for(name, (4, 19, 70), seed=31).values())
    prov = DecoderProvider.load(folders(name), dtype=dtype, max_batch=2, max_tokens=1024)
    outs = prov.generate([GenerationRequest(prompt_ids=p, max_tokens=12) for p in prompts])
    for p, out in zip(prompts, outs):
        assert len(out.token_ids) == 12 and out.finish_reason == "length"
        # every token the engine chose is, for the plain restatement given the same prefix, the best token or
        # within rounding of it
        seq = list(p)
        for tok in out.token_ids:
            ref = plain.forward(raw, w, seq)[-1]
            slack = (1e-4 if dtype == "float32" else 0.12) * float(ref.abs().max())
            assert float(ref.max() - ref[tok]) <= slack
            seq.append(tok)


def test_the_command_line_generates(folders):
    proc = subprocess.run([sys.executable, "-m", "esp_b200", "generate", "--model", str(folders("A")), "--dtype", "float32",
                           "--prompt-ids", "5,17,3", "--prompt-ids", "9 8 7 6 5 4", "--max-tokens", "5"],
                          capture_output=True, text=True, env=dict(os.environ), cwd=str(repo_root()), timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    lines = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    assert [len(l["token_ids"]) for l in lines] == [5, 5]
    raw, _, w = model("A")
    want, margins = plain.greedy(raw, w, [5, 17, 3], 5)
    if min(margins) > 1e-3:
        assert lines[0]["token_ids"] == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(folders, tmp_path, dtype):
    name = "B"                                     # its sparse layers choose every expert or sit behind margins
    reqs = requests_for(name, (1, 60, 141), seed=17)
    ids = list(reqs)
    steps = steps_tail(reqs, tail=20) + steps_batches({k + "x": v for k, v in reqs.items()}, [[i + "x" for i in ids]],
                                                      {i + "x": max(1, len(reqs[i]) - 9) for i in ids})
    lines, wanted = [], []
    for i, (entries, end) in enumerate(steps):
        lines.append(json.dumps({"step": i, "entries": [{"id": rid, "tokens": t, "want": wnt} for rid, t, wnt in entries],
                                 "end": end}))
        wanted.append(sum(len(wnt) for _, _, wnt in entries))
    proc = subprocess.run([sys.executable, str(repo_root() / "bin" / "trace_run"), "--model", str(folders(name)), "--dtype",
                           dtype, "--out", str(tmp_path), "--max-tokens", "404"], input="\n".join(lines) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert proc.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    vocab = model(name)[0]["vocab"]
    rec = Recorder(vocab)
    pos = {}
    for i, (entries, _end) in enumerate(steps):
        data = np.fromfile(tmp_path / f"{i}.f32", dtype="<f4").reshape(wanted[i], vocab)
        r = 0
        for rid, toks, want in entries:
            for wnt in want:
                rec.logits.setdefault(rid, {})[pos.get(rid, 0) + wnt] = data[r]
                r += 1
            pos[rid] = pos.get(rid, 0) + len(toks)
    both = dict(reqs)
    both.update({k + "x": v for k, v in reqs.items()})
    if dtype == "float32":
        check(name, dtype, both, rec, "replay program")
    else:
        # the program records no expert choices: hold its rows against an engine that does, which is held against
        # the plain restatement
        eng = engine_for(folders(name), dtype)
        other = Choices(vocab)
        run_steps(eng, steps, other)
        check(name, dtype, both, other, "replay program's steps in the engine")
        for rid, toks in both.items():
            at = list(range(len(toks)))
            assert np.array_equal(rec.logits_of(rid, at), other.logits_of(rid, at))
