"""The Pilutar decoder through the engine against the plain implementation (tests/plain_pilutar.py), in 32-bit and in
bfloat16, under every way of cutting the work: whole prompts from one token on, prompt then token by token across page
borders, windows' edges and the recurrence's chunk borders, token by token from the first, portions down to two tokens,
mixed batches of unequal requests on so few pages and slots that they are used again, long decoding, a far token that
only the recurrence can still know, keys just inside and just outside every window, replayed graphs, and greedy
generation through `generate()`, the scheduler and the command lines."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_pilutar
import pilutar_helpers as ph

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
MODELS = list(ph.PILUTAR)
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("pilutar")
    return {name: ph.make_model(str(root / name), name) for name in MODELS}


def make_engine(model, dtype, max_tokens, max_seqs=4, **more):
    from lia_rs_b200.engine import Engine
    return Engine(model["dir"], dtype=dtype, page_size=model["page_size"], max_tokens=max_tokens, max_seqs=max_seqs,
                  max_batch_tokens=max(256, max_tokens), **more)


def tokens_of(model, count, seed):
    return helpers.random_tokens(model["config"]["vocab"], count, seed)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_whole_prompts_and_first_tokens(models, name, dtype):
    model = models[name]
    engine = make_engine(model, dtype, 192)
    replay = helpers.Replayer(engine)
    for i, count in enumerate([1, 2, 3, 31, 32, 33, 65, 100, 170]):      # around the recurrence's chunks of 32 tokens and the windows
        tokens = tokens_of(model, count, 20 + i)
        logits = replay.step([("r", tokens, range(count))], end=["r"])
        ph.assert_close(logits, ph.plain_logits(model, tokens), dtype, f"{name} whole {count}", model["config"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_prompt_then_token_by_token(models, name, dtype):
    """The decoded tokens pass several page borders; the recurrent layers carry their state through every single step,
    the windows slide over the decoded tokens."""
    model = models[name]
    tokens = tokens_of(model, 150, 5)
    reference = ph.plain_logits(model, tokens)
    engine = make_engine(model, dtype, 192)
    replay = helpers.Replayer(engine)
    head = 37
    rows = [replay.step([("r", tokens[:head], [head - 1])])]
    for i in range(head, len(tokens)):
        rows.append(replay.step([("r", [tokens[i]], [0])]))
    ph.assert_close(np.concatenate(rows), reference[head - 1:], dtype, f"{name} decode", model["config"])
    # all of it token by token from the first token on, in the slot and the pages that the request above gives back
    replay.step([], end=["r"])
    rows = [replay.step([("s", [t], [0])]) for t in tokens[:60]]
    ph.assert_close(np.concatenate(rows), reference[:60], dtype, f"{name} token by token", model["config"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_portions_of_changing_size(models, name, dtype):
    model = models[name]
    tokens = tokens_of(model, 173, 8)
    reference = ph.plain_logits(model, tokens)
    for sizes in ([2, 2, 3, 2, 5, 1, 2, 7, 16, 2, 31, 1, 1, 2, 40, 3, 2, 51], [64, 2, 64, 2, 41], [3] * 40 + [53],
                  [32, 33, 31, 1, 64, 12]):
        engine = make_engine(model, dtype, 192)
        replay = helpers.Replayer(engine)
        rows, at = [], 0
        for size in sizes:
            rows.append(replay.step([("r", tokens[at:at + size], range(size))]))
            at += size
        assert at == len(tokens)
        ph.assert_close(np.concatenate(rows), reference, dtype, f"{name} portions {sizes[:4]}", model["config"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_mixed_batches_on_reused_pages_and_slots(models, name, dtype):
    """Four slots, five requests of unequal length, a pool that holds them only because finished requests give
    their pages back; portions beside single tokens; every request equals itself alone (the plain model).  The fifth
    request takes a slot whose recurrent state and pages another request has used: its state must start from zero."""
    model = models[name]
    lengths = {"a": 120, "b": 9, "c": 63, "d": 30, "e": 77}
    tokens = {r: tokens_of(model, n, 40 + i) for i, (r, n) in enumerate(lengths.items())}
    engine = make_engine(model, dtype, 256, max_seqs=4)
    replay = helpers.Replayer(engine)
    got = {r: [] for r in lengths}
    at = {r: 0 for r in lengths}
    plan = [
        [("a", 16), ("b", 2)], [("a", 29), ("b", 1), ("c", 5)], [("a", 1), ("b", 1), ("c", 40), ("d", 2)],
        [("a", 3), ("b", 5), ("c", 1), ("d", 28)], [("a", 64), ("c", 17)], [("e", 33), ("a", 1)],
        [("e", 1), ("a", 2)], [("e", 43), ("a", 4)],
    ]
    for step in plan:
        batch, ends = [], []
        for request, count in step:
            start = at[request]
            batch.append((request, tokens[request][start:start + count], range(count)))
            at[request] = start + count
            if at[request] == lengths[request]:
                ends.append(request)
        out = replay.step(batch, end=ends)
        row = 0
        for request, count in step:
            got[request].append(out[row:row + count])
            row += count
    for request, rows in got.items():
        assert at[request] == lengths[request]
        ph.assert_close(np.concatenate(rows), ph.plain_logits(model, tokens[request]), dtype,
                        f"{name} mixed {request}", model["config"])


@pytest.mark.parametrize("name", MODELS)
def test_ways_of_cutting_agree_in_32_bit(models, name):
    """Whole, portions and token by token give the same logits far inside the 32-bit tolerance."""
    model = models[name]
    tokens = tokens_of(model, 90, 3)
    outputs = []
    for sizes in ([90], [2] * 10 + [33, 37], [50] + [1] * 40):
        engine = make_engine(model, "float32", 128)
        replay = helpers.Replayer(engine)
        rows, at = [], 0
        for size in sizes:
            rows.append(replay.step([("r", tokens[at:at + size], range(size))]))
            at += size
        outputs.append(np.concatenate(rows))
    scale = np.abs(outputs[0]).max()
    for other in outputs[1:]:
        assert np.abs(other - outputs[0]).max() <= 3e-5 * scale


@pytest.mark.parametrize("cut", ["whole", "portions", "decode"])
@pytest.mark.parametrize("name", ["pil-A", "pil-C"])
def test_a_far_token_alone_decides(models, name, cut):
    """A sequence in which one token, 300 and more positions back and far outside every window, is the only one of its
    kind: the logits of the last positions with and without it differ by far more than the tolerance in the plain model
    (the recurrence's slow channels still hold it), so a state that forgot, was cleared or was carried wrongly across a
    chunk or a step would show.  32-bit."""
    model = models[name]
    vocab = model["config"]["vocab"]
    filler = helpers.random_tokens(vocab - 1, 340, 12)            # never the last id
    tokens = list(filler)
    tokens[7] = vocab - 1
    reference, without = ph.plain_logits(model, tokens), ph.plain_logits(model, filler)
    tail = slice(330, 340)
    assert float((reference[tail] - without[tail]).abs().max()) > 1e-3 * float(reference.abs().max())
    engine = make_engine(model, "float32", 384)
    replay = helpers.Replayer(engine)
    sizes = {"whole": [340], "portions": [5, 64, 31, 2, 130, 33, 75], "decode": [300] + [1] * 40}[cut]
    rows, at = [], 0
    for size in sizes:
        rows.append(replay.step([("r", tokens[at:at + size], range(size))]))
        at += size
    ph.assert_close(np.concatenate(rows)[tail], reference[tail], "float32", f"{name} far token, {cut}", model["config"])


@pytest.mark.parametrize("cut", ["whole", "portions", "decode"])
def test_keys_just_inside_and_just_outside_a_window(models, cut):
    """A model of latent attention alone (nothing but the windows carries anything from token to token): a token that
    is the only one of its kind changes the logits of the positions whose windows (widened layer by layer) still reach
    it, and of no position behind them.  The engine must agree with the plain model on both sides of that edge, in
    prompts, in portions and in decoding: a window that is one token too wide or too narrow shows.  32-bit."""
    model = models["pil-D"]
    vocab = model["config"]["vocab"]
    windows = [layer["mixer"]["mask"]["size"] for layer in model["config"]["layers"]]
    reach = sum(w - 1 for w in windows)                          # the farthest position that the marked token can touch
    at_token = 9
    filler = helpers.random_tokens(vocab - 1, at_token + reach + 12, 31)
    tokens = list(filler)
    tokens[at_token] = vocab - 1
    reference, without = ph.plain_logits(model, tokens), ph.plain_logits(model, filler)
    edge = at_token + reach
    scale = float(reference.abs().max())
    assert float((reference[at_token:edge + 1] - without[at_token:edge + 1]).abs().max()) > 1e-3 * scale      # inside
    assert float((reference[edge + 1:] - without[edge + 1:]).abs().max()) < 1e-9 * scale   # just outside
    engine = make_engine(model, "float32", 256)
    replay = helpers.Replayer(engine)
    n = len(tokens)
    sizes = {"whole": [n], "portions": [3, 17, 2, 40] + [n - 62], "decode": [at_token + 2] + [1] * (n - at_token - 2)}[cut]
    rows, at = [], 0
    for size in sizes:
        rows.append(replay.step([("r", tokens[at:at + size], range(size))]))
        at += size
    got = np.concatenate(rows)
    ph.assert_close(got, reference, "float32", f"window edge, {cut}", model["config"])
    # the edge row carries the marked token's trace, the row behind it does not: to the tolerance of the 32-bit path
    limit = 8.0 * ph.longest_sum(model["config"]) * 2.0 ** -24 * scale * len(windows)
    assert np.abs(got[edge + 1:] - without[edge + 1:].numpy()).max() <= limit


@pytest.mark.parametrize("seed", range(301, 313))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Twelve configurations drawn at random (layer order, every size, every optional key): whole, in portions beside
    another request's single tokens on reused pages, and token by token, in 32-bit against the plain model; whole and
    portions in bfloat16."""
    model = ph.make_model(str(tmp_path / "m"), f"random-{seed}")
    tokens, other = tokens_of(model, 83, seed), tokens_of(model, 21, seed + 1)
    reference, reference_other = ph.plain_logits(model, tokens), ph.plain_logits(model, other)
    for dtype in DTYPES:
        engine = make_engine(model, dtype, 128)
        replay = helpers.Replayer(engine)
        logits = replay.step([("w", tokens, range(len(tokens)))], end=["w"])
        ph.assert_close(logits, reference, dtype, f"random {seed} whole", model["config"])
        rows, others, at = [], [], 0
        for i, size in enumerate([2, 19, 1, 33, 5, 23]):
            batch = [("r", tokens[at:at + size], range(size))]
            if i < len(other) // 4:
                batch.append(("o", other[4 * i:4 * i + 4] if i % 2 else other[4 * i:4 * i + 1], range(4 if i % 2 else 1)))
            out = replay.step(batch)
            rows.append(out[:size])
            if len(batch) > 1:
                others.append(out[size:])
            at += size
        assert at == len(tokens)
        ph.assert_close(np.concatenate(rows), reference, dtype, f"random {seed} portions", model["config"])
        replay.step([], end=["r", "o"])
        if dtype == "float32":
            rows = [replay.step([("s", [t], [0])]) for t in tokens[:40]]
            ph.assert_close(np.concatenate(rows), reference[:40], dtype, f"random {seed} token by token", model["config"])


@pytest.mark.parametrize("name", ["pil-A", "pil-B"])
def test_long_decoding(models, name):
    """400 tokens one by one behind a short prompt, bfloat16: the state and the pages hold over hundreds of steps."""
    model = models[name]
    tokens = tokens_of(model, 420, 77)
    reference = ph.plain_logits(model, tokens)
    engine = make_engine(model, "bfloat16", 448)
    replay = helpers.Replayer(engine)
    rows = [replay.step([("r", tokens[:20], [19])])]
    rows += [replay.step([("r", [t], [0])]) for t in tokens[20:]]
    ph.assert_close(np.concatenate(rows), reference[19:], "bfloat16", f"{name} long decode", model["config"])


@pytest.mark.parametrize("name", ["pil-A", "pil-D"])
def test_graphs_replay_what_was_launched(models, name):
    """Steps replayed as CUDA graphs against steps launched kernel by kernel, to the bit (bfloat16)."""
    model = models[name]
    tokens = tokens_of(model, 120, 9)
    outputs = []
    for graphs in (True, False):
        engine = make_engine(model, "bfloat16", 256, cuda_graphs=graphs)
        rows = []
        for _ in range(3 if graphs else 1):
            replay = helpers.Replayer(engine)
            rows = [replay.step([("r", tokens[:40], [39])]), replay.step([("r", tokens[40:80], [39])])]
            rows += [replay.step([("r", [t], [0])]) for t in tokens[80:]]
            replay.step([], end=["r"])
        if graphs:
            assert engine.cuda_graphs and engine.stats["graph_replays"] > 40
        outputs.append(np.concatenate(rows))
    assert np.array_equal(outputs[0], outputs[1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["pil-A", "pil-B", "pil-D"])
def test_greedy_generation_through_generate_and_the_scheduler(models, name, dtype):
    from lia_rs_b200 import generate
    model = models[name]
    prompts = [tokens_of(model, n, 60 + i) for i, n in enumerate((5, 19, 33, 2, 47))]
    count = 12
    got = generate(model["dir"], prompts, max_tokens=count, dtype=dtype, page_size=model["page_size"],
                   kv_pool_tokens=192, max_sequences=3, prefill_batch=16)       # 5 requests over 3 slots, portions of 16
    for prompt, tokens in zip(prompts, got):
        assert len(tokens) == count
        # rounding may turn a near tie: each token must be a maximum of the plain model's logits for the sequence it
        # continues, within the rounding of that path
        logits = ph.plain_logits(model, list(prompt) + tokens)
        slack = 2e-4 if dtype == "float32" else 5e-2
        for i, token in enumerate(tokens):
            row = logits[len(prompt) - 1 + i]
            assert float(row.max() - row[token]) <= slack * max(1.0, float(row.abs().max())), (name, i, token)
    if dtype == "float32":
        want = [plain_pilutar.greedy(model["config"], model["weights"], p, count) for p in prompts[:2]]
        agree = sum(g == w for g, w in zip(got[:2], want))
        assert agree >= 1          # (a near tie may turn one of them; both turning would be a fault)


def test_trace_runner_and_command_line(models, tmp_path):
    """bin/trace_run replays a trace of two requests on a small pool; `lia inspect` names the architecture and
    `lia forward-batch` gives the plain model's greedy choice at every position."""
    model = models["pil-A"]
    a, b = tokens_of(model, 30, 1), tokens_of(model, 11, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[7:9], "want": [0, 1]}, {"id": "b", "tokens": b, "want": [10]}],
              "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[9:], "want": [20]}], "end": ["a"]}]
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model["dir"], "--dtype",
                           "float32", "--out", str(out), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    vocab = model["config"]["vocab"]
    ref_a, ref_b = ph.plain_logits(model, a), ph.plain_logits(model, b)
    rows = {s: np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, vocab) for s in (0, 1, 2)}
    ph.assert_close(rows[0], ref_a[6:7], "float32", "trace step 0", model["config"])
    ph.assert_close(rows[1], torch.cat([ref_a[7:9], ref_b[10:11]]), "float32", "trace step 1", model["config"])
    ph.assert_close(rows[2], ref_a[29:30], "float32", "trace step 2", model["config"])
    lia = [sys.executable, os.path.join(ROOT, "bin", "lia")]
    shown = subprocess.run(lia + ["inspect", model["dir"]], capture_output=True, text=True, timeout=300)
    assert shown.returncode == 0 and "architecture=Pilutar" in shown.stdout and "tensor l1.mlp.router" in shown.stdout and \
        "tensor l0.mix.right.a2.b" in shown.stdout
    batch = subprocess.run(lia + ["forward-batch", model["dir"], ",".join(map(str, b)), "--dtype", "float32"],
                           capture_output=True, text=True, timeout=900)
    assert batch.returncode == 0, batch.stderr[-2000:]
    chosen = [int(line.split("token=")[1].split()[0]) for line in batch.stdout.splitlines() if line.startswith("position=")]
    assert chosen == [int(torch.where(row == row.max())[0].max()) for row in ref_b]
