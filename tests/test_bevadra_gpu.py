"""The Bevadra design through the framework against the plain implementation of ``plain_bevadra.py``: each
mechanism alone, whole prompts against portions and token-by-token decoding, mixed batches with pages that are used
again, window edges with keys that stand out, long decoding, several sizes, and greedy generation through the
engine's entry point."""

from __future__ import annotations

import json
import math
import random
from pathlib import Path

import pytest
import torch

import plain_bevadra as plain
import schedules
from conftest import note_error

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# Largest |engine - plain| relative to the request's largest |logit|.
TOLERANCE = {"float32": 2e-5, "bfloat16": 5e-2}


def attention(heads, kv_heads, dim, vdim, scale, window, kv_from=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        out["mask"] = {"size": window}
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, window, base, dims=None):
    out = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
           "rot": {"base": base, "dims": rot_dim if dims is None else dims}}  # fmt: skip
    if window:
        out["mask"] = {"size": window}
    return out


def dense(ff):
    return {"kind": "dense", "ff": ff}


# Five layers that differ from one another: a latent layer first; an attention layer whose keys and values a later
# layer reads with a wider window of its own; value heads wider and narrower than key heads; groups of three, one and
# two heads; layers without feed-forward; a latent layer that rotates only a part of its rotated elements.
CONFIG_S = {
    "architecture": "Bevadra", "vocab": 90, "width": 48, "norm": {"eps": 2e-5}, "logit_softcap": 6.0,
    "layers": [
        {"type": "latent_attention", "mixer": latent(3, 16, 8, 24, 20, 28, 0.2, 19, 300.0), "mlp": dense(40)},
        {"type": "attention", "mixer": attention(6, 2, 16, 24, 0.2, 20), "mlp": dense(24)},
        {"type": "latent_attention", "mixer": latent(2, 24, 12, 8, 36, 16, 0.15, 50, 10000.0, dims=8), "mlp": None},
        {"type": "attention", "mixer": attention(6, 2, 16, 24, 0.35, 33, kv_from=1), "mlp": dense(16)},
        {"type": "attention", "mixer": attention(2, 2, 24, 8, 0.15, 7), "mlp": None},
    ],
}  # fmt: skip
# Widths that the tensor-core products take, windows that straddle pages of 16, an attention layer without a window
# whose heads are 64 wide (keys and values alike), read again by a later layer with a window; a latent layer without a
# window; no soft cap.
CONFIG_T = {
    "architecture": "Bevadra", "vocab": 64, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": attention(8, 2, 32, 32, 0.18, 33), "mlp": dense(64)},
        {"type": "attention", "mixer": attention(2, 1, 64, 64, 0.125, None), "mlp": dense(32)},
        {"type": "latent_attention", "mixer": latent(4, 32, 16, 32, 64, 48, 0.14, None, 50000.0), "mlp": dense(64)},
        {"type": "attention", "mixer": attention(4, 1, 64, 64, 0.125, 16, kv_from=1), "mlp": None},
        {"type": "latent_attention", "mixer": latent(8, 16, 32, 16, 32, 64, 0.2, 17, 100.0), "mlp": dense(128)},
    ],
}  # fmt: skip
# Sizes that no fast path takes: a width that is no multiple of 8, odd head widths, one head, windows of one token,
# ranks of one and of an odd number, a rotated part of two elements.
CONFIG_U = {
    "architecture": "Bevadra", "vocab": 51, "width": 36, "norm": {"eps": 1e-4}, "logit_softcap": 30.0,
    "layers": [
        {"type": "attention", "mixer": attention(1, 1, 10, 6, 0.4, 1), "mlp": dense(17)},
        {"type": "latent_attention", "mixer": latent(1, 5, 2, 7, 1, 3, 0.5, 1, 20.0), "mlp": dense(9)},
        {"type": "attention", "mixer": attention(3, 1, 14, 20, 0.3, 9), "mlp": None},
        {"type": "latent_attention", "mixer": latent(5, 6, 10, 3, 13, 11, 0.3, 23, 1000.0, dims=6), "mlp": None},
    ],
}  # fmt: skip
CONFIGS = {"S": CONFIG_S, "T": CONFIG_T, "U": CONFIG_U}
LENGTHS = {"S": [70, 45, 133, 9, 97, 33, 1, 2], "T": [150, 64, 17, 81, 49, 130], "U": [40, 3, 77, 18, 1, 60]}


def random_ids(seed, count, vocab):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]


def write_model(folder, raw, seed=31, scale=12.0):
    from mini_engine_b200.config import BevadraConfig
    from mini_engine_b200.weights import write_random_model

    write_random_model(folder, BevadraConfig.from_dict(raw), seed=seed, dtype=torch.bfloat16, scale=scale)
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_model(tmp_path_factory.mktemp(f"bevadra_{name}"), raw) for name, raw in CONFIGS.items()}


def load_plain(folder):
    from safetensors.torch import load_file

    weights = {k: v.to(torch.float64) for k, v in load_file(str(Path(folder) / "model.safetensors")).items()}
    return weights, json.loads((Path(folder) / "config.json").read_text())


def expected_logits(folder, requests):
    weights, config = load_plain(folder)
    return {name: plain.forward(config, weights, toks).float() for name, toks in requests.items()}


def replay(folder, dtype_name, steps, block_size=16, max_tokens=None, max_live=4, max_step_tokens=512):
    from mini_engine_b200.engine.replay import Replayer

    replayer = Replayer(folder, DTYPES[dtype_name], max_tokens or schedules.peak_live_tokens(steps), block_size,
                        max_step_tokens=max_step_tokens, max_live=max_live)  # fmt: skip
    outputs = {}
    for record in steps:
        logits = replayer.step(record)
        if logits is not None:
            outputs[record["step"]] = logits.clone()
    replayer.manager.check_invariants([])
    assert all(pool.num_free == pool.num_pages for pool in replayer.manager.pools), "pages were lost"
    return schedules.collect(steps, outputs)


def compare(got, expected, requests, dtype_name):
    worst = 0.0
    for name, toks in requests.items():
        assert sorted(got[name]) == list(range(len(toks))), f"{name}: positions missing"
        scale = float(expected[name].abs().max())
        for position, row in got[name].items():
            error = float((row - expected[name][position]).abs().max()) / scale
            worst = max(worst, error)
            assert error <= TOLERANCE[dtype_name], f"{name} position {position}: relative error {error:.3g}"
    note_error("bevadra " + dtype_name, worst)


def replay_and_compare(folder, dtype_name, steps, requests, **options):
    compare(replay(folder, dtype_name, steps, **options), expected_logits(folder, requests), requests, dtype_name)


def requests_for(name):
    return {f"r{i}": random_ids(500 + i, n, CONFIGS[name]["vocab"]) for i, n in enumerate(LENGTHS[name])}


# --------------------------------------------------------------- whole models, every way of cutting


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["S", "T", "U"])
@pytest.mark.parametrize("schedule", ["whole", "tail_one_by_one", "changing_portions", "mixed"])
def test_schedules_match_plain(name, dtype_name, schedule, folders):
    """Whole prompts (requests of one and two tokens among them); the last 32 tokens one by one (the windows pass
    over decoded tokens); portions down to two tokens; up to four live requests whose pages are handed out again."""
    requests = requests_for(name)
    steps = getattr(schedules, schedule)(requests)
    replay_and_compare(folders[name], dtype_name, steps, requests)


UNUSUAL = {
    # two readers of one owner that has no window itself: one with a window shorter than a page, one with a long one
    "readers_of_one_owner": [
        {"type": "attention", "mixer": attention(4, 1, 64, 64, 0.125, None), "mlp": None},
        {"type": "attention", "mixer": attention(4, 1, 64, 64, 0.125, 10, kv_from=0), "mlp": dense(64)},
        {"type": "attention", "mixer": attention(4, 1, 64, 64, 0.3, 200, kv_from=0), "mlp": None},
    ],
    # only latent layers: every cache row serves as key and as value; two layers of equal sizes share a cache group
    "only_latent": [
        {"type": "latent_attention", "mixer": latent(4, 16, 16, 16, 48, 32, 0.2, 40, 10000.0), "mlp": dense(32)},
        {"type": "latent_attention", "mixer": latent(4, 16, 16, 16, 48, 32, 0.2, 40, 10000.0), "mlp": None},
        {"type": "latent_attention", "mixer": latent(2, 64, 64, 128, 128, 96, 0.08, None, 500.0), "mlp": dense(64)},
    ],
    # head sizes 128 with groups of four: what a full-size model has
    "wide_heads": [
        {"type": "attention", "mixer": attention(4, 1, 128, 128, 0.09, 48), "mlp": dense(64)},
        {"type": "attention", "mixer": attention(8, 2, 64, 64, 0.125, 100), "mlp": dense(64)},
    ],
}


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(UNUSUAL))
def test_unusual_layer_combinations(name, dtype_name, tmp_path):
    raw = {"architecture": "Bevadra", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 20.0, "layers": UNUSUAL[name]}
    write_model(tmp_path, raw, seed=5, scale=6.0)
    requests = {"a": random_ids(1, 300, 200), "b": random_ids(2, 77, 200), "c": random_ids(3, 1, 200), "d": random_ids(4, 2, 200)}
    for maker in (schedules.whole, schedules.changing_portions, schedules.mixed, lambda r: schedules.tail_one_by_one(r, 32)):
        replay_and_compare(tmp_path, dtype_name, maker(requests), requests)


@pytest.mark.parametrize("block_size", [4, 16, 32])
def test_float32_does_not_depend_on_the_cut_or_the_batch(folders, block_size):
    """In float32 every kernel's sums for a token depend on that token's position alone, so portions, single
    tokens, mixed batches and other page sizes give the whole prompt's bits."""
    requests = {name: toks for name, toks in list(requests_for("S").items())[:5]}
    whole = replay(folders["S"], "float32", schedules.whole(requests), block_size)
    for maker in (schedules.changing_portions, schedules.mixed, lambda r: schedules.tail_one_by_one(r, 40)):
        cut = replay(folders["S"], "float32", maker(requests), block_size)
        for name, toks in requests.items():
            for position in range(len(toks)):
                assert torch.equal(whole[name][position], cut[name][position]), f"{name} position {position}"


def test_long_decoding_past_every_window(folders):
    """Three prompt tokens, then 200 tokens one by one: the windows are all that is left of the start."""
    for name in ("S", "T"):
        requests = {"long": random_ids(77, 203, CONFIGS[name]["vocab"])}
        steps = schedules.tail_one_by_one(requests, tail=200)
        for dtype_name in ("float32", "bfloat16"):
            replay_and_compare(folders[name], dtype_name, steps, requests)


def test_pages_that_are_used_again_hold_nothing_of_their_past(folders):
    """A pool of four pages: the second request gets the first one's pages and must not see what they held."""
    from mini_engine_b200.engine.replay import Replayer

    a, b = random_ids(5, 60, CONFIG_S["vocab"]), random_ids(6, 37, CONFIG_S["vocab"])
    replayer = Replayer(folders["S"], torch.float32, 64, 16, max_live=1)
    first = replayer.step({"step": 0, "entries": [{"id": "a", "tokens": a, "want": [59]}], "end": ["a"]})
    assert replayer.step({"step": 1, "entries": [{"id": "b", "tokens": b[:20], "want": []}], "end": []}) is None
    second = replayer.step({"step": 2, "entries": [{"id": "b", "tokens": b[20:], "want": [16]}], "end": ["b"]})
    alone = Replayer(folders["S"], torch.float32, 64, 16).step({"step": 0, "entries": [{"id": "b", "tokens": b, "want": [36]}], "end": ["b"]})
    assert torch.equal(second, alone) and not torch.equal(first, alone)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_the_replay_program_itself(folders, dtype_name, tmp_path):
    """`bin/trace_run` as a process on a model folder of this design: mixed steps in, `done` lines and logit files out."""
    import subprocess
    import sys

    import numpy as np
    from conftest import ROOT

    requests = requests_for("U")
    steps = schedules.mixed(requests)
    out = tmp_path / "out"
    feed = "".join(json.dumps(record) + "\n" for record in steps)
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders["U"]), "--dtype", dtype_name,
         "--out", str(out), "--max-tokens", str(schedules.peak_live_tokens(steps))],
        input=feed, capture_output=True, text=True, timeout=900,
    )  # fmt: skip
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    outputs = {}
    for record in steps:
        wanted = sum(len(e.get("want", [])) for e in record["entries"])
        if wanted:
            data = np.fromfile(out / f"{record['step']}.f32", dtype="<f4")
            outputs[record["step"]] = torch.from_numpy(data.reshape(wanted, CONFIG_U["vocab"]).copy())
    got = schedules.collect(steps, outputs)
    compare(got, expected_logits(folders["U"], requests), requests, dtype_name)


def test_the_stream_after_every_layer(folders):
    """The residual stream behind each layer (the stream plus everything that is still to be added) against the
    plain layers, in float32."""
    from mini_engine_b200.engine.replay import Replayer
    from mini_engine_b200.parts import block as block_module

    weights, config = load_plain(folders["S"])
    toks = random_ids(9, 50, config["vocab"])
    _, want = plain.forward(config, weights, toks, return_layers=True)
    seen = []
    original = block_module.ParallelBlock.forward

    def recording(self, state, ctx, cache):
        original(self, state, ctx, cache)
        x = state.x.clone() + state.pending.sum(0)
        if state.pending_bias is not None:
            x += state.pending_bias
        if state.pending_more is not None:
            x += state.pending_more.sum(0)
        seen.append(x)

    block_module.ParallelBlock.forward = recording
    try:
        Replayer(folders["S"], torch.float32, 64).step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": ["a"]})
    finally:
        block_module.ParallelBlock.forward = original
    assert len(seen) == len(config["layers"])
    for index, got in enumerate(seen):
        assert torch.allclose(got.cpu(), want[index].float(), atol=2e-5 * float(want[index].abs().max())), f"layer {index}"


# ---------------------------------------------------------------------- mechanisms alone: small kernels


def cuda(t, dtype=None):
    return None if t is None else t.to(device="cuda", dtype=dtype or t.dtype).contiguous()


@pytest.mark.parametrize("hidden", [36, 48, 256, 1000])
def test_sum_and_layer_norm(hidden):
    """x + bias + the partial sums of two sublayers, then the layer norm; all rows, and chosen rows without touching x."""
    from mini_engine_b200.csrc import ops

    torch.manual_seed(hidden)
    T = 9
    x = torch.randn(T, hidden) * 3 + 5.0  # a mean far from zero: the variance is taken around it
    first, second = torch.randn(3, T, hidden), torch.randn(2, T, hidden)
    add_bias, weight, bias = torch.randn(hidden), torch.randn(hidden), torch.randn(hidden)
    total = x.double() + first.double().sum(0) + add_bias.double() + second.double().sum(0)
    want = plain.layer_norm(total, weight.double(), bias.double(), 1e-5)
    for dtype, tolerance in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        stream, out = cuda(x), torch.empty(T, hidden, dtype=dtype, device="cuda")
        ops.add_layernorm(stream, cuda(first), cuda(weight), cuda(bias), 1e-5, out, None, cuda(second), cuda(add_bias))
        assert torch.allclose(stream.cpu().double(), total, atol=1e-5)
        assert torch.allclose(out.float().cpu().double(), want, atol=tolerance * float(want.abs().max()))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    stream, out = cuda(x), torch.empty(3, hidden, dtype=torch.float32, device="cuda")
    ops.add_layernorm(stream, cuda(first), cuda(weight), cuda(bias), 1e-5, out, cuda(rows), cuda(second), cuda(add_bias))
    assert torch.equal(stream.cpu(), x)
    assert torch.allclose(out.cpu().double(), want[rows.long()], atol=1e-5 * float(want.abs().max()))
    # nothing pending: the plain norm of x, which stays as it is
    ops.add_layernorm(stream, None, cuda(weight), cuda(bias), 1e-5, out, cuda(rows))
    assert torch.allclose(out.cpu().double(), plain.layer_norm(x.double(), weight.double(), bias.double(), 1e-5)[rows.long()], atol=1e-5 * float(want.abs().max()))


@pytest.mark.parametrize("inter", [17, 64])
def test_gated_unit_with_the_tanh_gelu(inter):
    from mini_engine_b200.csrc import ops

    torch.manual_seed(inter)
    both = torch.randn(2, 11, 2 * inter) * 2
    whole = both.double().sum(0)
    want = plain.gelu_tanh(whole[:, :inter]) * whole[:, inter:]
    out = torch.empty(11, inter, dtype=torch.float32, device="cuda")
    ops.swiglu(cuda(both), out, activation="gelu_tanh")
    assert torch.allclose(out.cpu().double(), want, atol=1e-5)
    ops.swiglu(cuda(both), out)  # the default is still the sigmoid gate
    silu = whole[:, :inter] * torch.sigmoid(whole[:, :inter]) * whole[:, inter:]
    assert torch.allclose(out.cpu().double(), silu, atol=1e-5)


# ---------------------------------------------------------------------- mechanisms alone: attention


def paged(rows, page_size, pages_total, generator):
    """``rows [T, kv, d]`` -> page array ``[pages_total + 1, kv, page_size, d]`` with the request's pages in
    shuffled places and the rest filled with large numbers, and the block table."""
    T, kv, d = rows.shape
    count = -(-T // page_size)
    order = torch.randperm(pages_total, generator=generator)[:count]
    pages = torch.full((pages_total + 1, kv, page_size, d), 1e4, dtype=rows.dtype)
    for t in range(T):
        pages[order[t // page_size], :, t % page_size] = rows[t]
    return pages, order.to(torch.int32)


def plain_biased_attention(q, k, v, scale, window, slopes=None, sink=None, gate=None):
    """[T, H, V]: the attention mixer's core from the plain module's pieces (float64)."""
    T, H, _ = q.shape
    rep = H // k.shape[1]
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    pos = torch.arange(T, dtype=q.dtype)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if slopes is not None:
        scores = scores - slopes.to(q.dtype).view(-1, 1, 1) * (pos.view(-1, 1) - pos.view(1, -1))
    weights = plain.softmax_with_extra(scores, plain.window_mask(T, window, q), None if sink is None else sink.to(q.dtype))
    out = torch.einsum("hij,jhd->ihd", weights, vv)
    return out if gate is None else out * gate.to(q.dtype).view(T, H, -1)


def run_attention(q, k, v, scale, window, positions, dtype, page_size=16, slopes=None, sink=None, gate=None, through=None):
    """The generic attention kernel on one request whose keys 0..T-1 are cached; ``v=None``: the values are the
    first ``value_dim`` elements of the key rows."""
    from mini_engine_b200.csrc import ops

    T, G, D = k.shape
    H = q.shape[1]
    V = v.shape[2] if v is not None else through
    generator = torch.Generator().manual_seed(T)
    k_pages, table = paged(k, page_size, 3 * (-(-T // page_size)), generator)
    v_pages = None
    if v is not None:
        generator.manual_seed(T)
        v_pages, _ = paged(v, page_size, 3 * (-(-T // page_size)), generator)
    n = len(positions)
    out = torch.empty(n, H * V, dtype=dtype, device="cuda")
    ops.paged_attention_generic(
        cuda(q[positions].reshape(n, H * D), dtype), cuda(k_pages, dtype), cuda(v_pages, dtype), cuda(table.view(1, -1)),
        torch.zeros(n, dtype=torch.int32, device="cuda"), torch.tensor(positions, dtype=torch.int32, device="cuda"), out,
        H, G, D, scale, window or 0, value_dim=V, gate=cuda(None if gate is None else gate[positions], torch.float32),
        slopes=cuda(slopes, torch.float32), sink_values=cuda(sink, torch.float32),
    )  # fmt: skip
    torch.cuda.synchronize()
    return out.float().cpu().view(n, H, V)


def slopes_of(heads, span=8.0):
    return torch.tensor([2.0 ** (-span * (h + 1) / heads) for h in range(heads)])


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 16, 8), (6, 3, 40, 72), (3, 1, 10, 33), (2, 2, 128, 128), (1, 1, 4, 1)])
@pytest.mark.parametrize("window", [None, 1, 16, 23])
def test_attention_with_bias_sink_and_element_gate_alone(heads, kv_heads, dim, vdim, window):
    torch.manual_seed(heads * 100 + dim)
    T = 75
    q, k, v = torch.randn(T, heads, dim), torch.randn(T, kv_heads, dim), torch.randn(T, kv_heads, vdim)
    gate, sink = torch.rand(T, heads * vdim), torch.randn(heads) * 2
    everyone = list(range(T))
    qd, kd, vd = q.double(), k.double(), v.double()
    want = plain_biased_attention(qd, kd, vd, 0.3, window, slopes_of(heads), sink, gate).float()
    got = run_attention(q, k, v, 0.3, window, everyone, torch.float32, slopes=slopes_of(heads), sink=sink, gate=gate)
    assert torch.allclose(got, want, atol=2e-5, rtol=2e-5)
    # each option alone changes the result, and is what the plain form says
    bare = run_attention(q, k, v, 0.3, window, everyone, torch.float32)
    assert torch.allclose(bare, plain_biased_attention(qd, kd, vd, 0.3, window).float(), atol=2e-5, rtol=2e-5)
    for options in ({"slopes": slopes_of(heads)}, {"sink": sink}, {"gate": gate}):
        alone = run_attention(q, k, v, 0.3, window, everyone, torch.float32, **options)
        assert torch.allclose(alone, plain_biased_attention(qd, kd, vd, 0.3, window, **options).float(), atol=2e-5, rtol=2e-5)
        if not (window == 1 and "slopes" in options):  # a query that sees only itself has no distance
            assert not torch.equal(alone, bare)
    # a sink far above every score takes all the weight; one far below leaves an ordinary softmax
    high = run_attention(q, k, v, 0.3, window, everyone, torch.float32, sink=torch.full((heads,), 200.0))
    assert float(high.abs().max()) < 1e-12
    low = run_attention(q, k, v, 0.3, window, everyone, torch.float32, sink=torch.full((heads,), -200.0))
    assert torch.allclose(low, bare, atol=2e-5, rtol=2e-5)


def test_the_distance_bias_grows_with_the_distance_not_with_the_position():
    """Equal keys everywhere: the weights then follow the bias alone, and with a sink they depend on the distance
    (a bias on the key's position alone would give the same softmax only without the sink)."""
    T, H, D = 60, 2, 8
    q, k = torch.ones(T, H, D), torch.ones(T, 1, D)
    v = torch.zeros(T, 1, T)
    v[torch.arange(T), 0, torch.arange(T)] = 1.0  # the output is the weight of every key
    slopes, sink = torch.tensor([0.5, 0.05]), torch.tensor([8.0 * 0.3, 8.0 * 0.3])  # the sink stands level with a key at distance 0
    got = run_attention(q, k, v, 0.3, None, [T - 1, 20], torch.float32, slopes=slopes, sink=sink)
    for row, position in enumerate((T - 1, 20)):
        for h in range(H):
            weights = got[row, h]
            expect = torch.exp(-slopes[h] * (position - torch.arange(position + 1).float()))
            expect = expect / (expect.sum() + 1.0)
            assert torch.allclose(weights[: position + 1], expect, atol=1e-6)
            assert float(weights[position + 1 :].abs().max() if position + 1 < T else 0.0) == 0.0


@pytest.mark.parametrize("window", [5, 16, 17, 31, 64])
@pytest.mark.parametrize("offset", ["just_inside", "just_outside", "far", "itself"])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["biased", "latent_rows"])
def test_a_key_that_stands_out_at_the_windows_edge(window, offset, dtype_name, kind):
    """One key has a score far above all others and a value that nothing else has: the query's output holds it
    exactly when the key lies inside the window, for a query in a prompt and for one decoded alone, over shuffled
    pages whose free places hold large numbers.  ``latent_rows``: one shared head whose values are the first elements
    of its key rows."""
    torch.manual_seed(window)
    T, H, D, V = 150, 4, 16, 12
    G = 2 if kind == "biased" else 1
    query = 140
    target = {"just_inside": query - window + 1, "just_outside": query - window, "far": 3, "itself": query}[offset]
    q, k = 0.1 * torch.randn(T, H, D), 0.1 * torch.randn(T, G, D)
    k[:, :, 0] = 0.0  # element 0 marks the target: no other key has it
    q[:, :, 0] = 0.0
    k[target] += 4.0 * q[query, 0] / q[query, 0].norm()  # aligned with head 0's query
    q[query] = 6.0 * q[query] / q[query].norm(dim=-1, keepdim=True)
    k[target, :, 0] = 100.0
    v = None if kind == "latent_rows" else torch.cat((k[:, :, :1], torch.randn(T, G, V - 1)), dim=-1)
    options = {"slopes": 0.01 * slopes_of(H), "sink": torch.zeros(H)} if kind == "biased" else {"through": V}
    visible = 0 <= query - target < window
    dtype = DTYPES[dtype_name]
    if dtype_name == "bfloat16":
        q, k = q.to(torch.bfloat16).float(), k.to(torch.bfloat16).float()
        v = None if v is None else v.to(torch.bfloat16).float()
    values = k[:, :, :V] if v is None else v
    want = plain_biased_attention(q.double(), k.double(), values.double(), 1.0, window, options.get("slopes"), options.get("sink")).float()
    for positions in ([query], list(range(query - 20, query + 5))):
        got = run_attention(q, k, v, 1.0, window, positions, dtype, **options)
        row = got[positions.index(query)]
        assert (row[0, 0] > 50.0) == visible, f"the marked value is {'missing' if visible else 'seen'}"
        tolerance = 2e-5 if dtype_name == "float32" else 2e-2
        assert torch.allclose(got, want[positions], atol=tolerance * 100.0, rtol=tolerance)


@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("heads,kv_heads,page", [(4, 2, 8), (8, 1, 16), (12, 1, 16), (4, 4, 4)])
@pytest.mark.parametrize("news", [[1, 1, 1, 1], [90, 5, 130, 2], [1, 40, 1, 7]])
@pytest.mark.parametrize("window", [0, 70])
def test_tensor_core_attention_with_bias_sinks_and_element_gates(head_dim, heads, kv_heads, page, news, window):
    """The bfloat16 kernels on tensor cores (prompt portions; decode by TMA for groups up to 8 and pages from 8
    tokens, else the tiled one; mixed steps) with the distance bias, learned sinks and a gate per element, against
    float64."""
    from test_kernels_gpu import fake_context

    from mini_engine_b200.csrc import attention_bf16, ops

    g = torch.Generator().manual_seed(head_dim + heads + page + len(news) + window)
    lengths = [400, 90, 130, 300]
    total_pages = sum(-(-n // page) for n in lengths) + 3
    order = torch.randperm(total_pages, generator=g).tolist()
    k_pages = torch.randn(total_pages, kv_heads, page, head_dim, generator=g).to(torch.bfloat16)
    v_pages = torch.randn(total_pages, kv_heads, page, head_dim, generator=g).to(torch.bfloat16)
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths) + 1), -1, dtype=torch.int32)
    slopes = 20.0 * slopes_of(heads)  # steep enough that the nearest keys carry the weight of the first heads
    sink = 3.0 * torch.randn(heads, generator=g)
    q_rows, want_rows, gate_rows, entry_of, positions = [], [], [], [], []
    for b, (n, new) in enumerate(zip(lengths, news)):
        q = (0.5 * torch.randn(n, heads, head_dim, generator=g)).to(torch.bfloat16)
        k = torch.randn(n, kv_heads, head_dim, generator=g).to(torch.bfloat16)
        v = torch.randn(n, kv_heads, head_dim, generator=g).to(torch.bfloat16)
        gate = torch.rand(n, heads * head_dim, generator=g)
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
        for p in range(n):
            k_pages[table[b, p // page], :, p % page] = k[p]
            v_pages[table[b, p // page], :, p % page] = v[p]
        want = plain_biased_attention(q.double(), k.double(), v.double(), head_dim**-0.5, window or None, slopes, sink, gate)
        q_rows.append(q[n - new :]), want_rows.append(want[n - new :]), gate_rows.append(gate[n - new :])
        entry_of += [b] * new
        positions += list(range(n - new, n))
    data = dict(new_counts=news, lengths=lengths, entry_of=torch.tensor(entry_of, dtype=torch.int32).cuda(),
                positions=torch.tensor(positions, dtype=torch.int32).cuda())  # fmt: skip
    q_all = torch.cat(q_rows).reshape(-1, heads * head_dim).contiguous().cuda()
    want = torch.cat(want_rows).reshape(-1, heads * head_dim).float()
    out = torch.full_like(q_all, float("nan"))
    assert attention_bf16.supports(head_dim, heads, kv_heads)
    ops.paged_attention(
        q=q_all, k_pages=k_pages.cuda(), v_pages=v_pages.cuda(), block_table=table.cuda(), ctx=fake_context(data), out=out,
        heads=heads, kv_heads=kv_heads, head_dim=head_dim, scale=head_dim**-0.5, window=window,
        gate=torch.cat(gate_rows).contiguous().cuda(), slopes=slopes.cuda(), sink_values=sink.cuda(),
    )  # fmt: skip
    torch.cuda.synchronize()
    assert attention_bf16.take_error() == 0
    error = float((out.float().cpu() - want).abs().max()) / float(want.abs().max())
    assert error < 2e-2, f"relative error {error:.3g}"


@pytest.mark.parametrize("heads,kv_heads,page", [(4, 2, 8), (6, 2, 16), (3, 1, 32), (2, 2, 128)])
@pytest.mark.parametrize("news", [[400, 90, 130, 300], [129, 33, 128, 2], [257, 1, 40, 256]])
@pytest.mark.parametrize(
    "which,window",
    [("all", w) for w in (0, 1, 70, 128, 200, 257)] + [("window_only", w) for w in (1, 70, 128, 200, 257)]
    + [(one, w) for one in ("bias", "sink", "gate_per_head") for w in (0, 200)],
)  # fmt: skip
def test_tensor_memory_attention_with_a_window_and_the_options(heads, kv_heads, page, news, window, which):
    """Prompt portions of 32 tokens and more with heads of 128 run with both products on tcgen05: windows that end
    inside, at the edge of and several tiles behind a block's first row, each option alone and all together, pages
    behind the window given back (their table entries are -1 and their contents large numbers), against float64."""
    from test_kernels_gpu import fake_context

    from mini_engine_b200.csrc import attention_bf16, ops

    head_dim = 128
    g = torch.Generator().manual_seed(heads + page + len(news) + window + news[0])
    lengths = [400, 90, 130, 300]
    total_pages = sum(-(-n // page) for n in lengths) + 3
    order = torch.randperm(total_pages, generator=g).tolist()
    k_pages = torch.full((total_pages, kv_heads, page, head_dim), 3e4).to(torch.bfloat16)
    v_pages = torch.full((total_pages, kv_heads, page, head_dim), -3e4).to(torch.bfloat16)
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths) + 1), -1, dtype=torch.int32)
    slopes = 20.0 * slopes_of(heads) if which in ("all", "bias") else None
    sink = 3.0 * torch.randn(heads, generator=g) if which in ("all", "sink") else None
    q_rows, want_rows, gate_rows, entry_of, positions = [], [], [], [], []
    for b, (n, new) in enumerate(zip(lengths, news)):
        q = (0.5 * torch.randn(n, heads, head_dim, generator=g)).to(torch.bfloat16)
        k = torch.randn(n, kv_heads, head_dim, generator=g).to(torch.bfloat16)
        v = torch.randn(n, kv_heads, head_dim, generator=g).to(torch.bfloat16)
        gate = {"all": torch.rand(n, heads * head_dim, generator=g), "gate_per_head": torch.rand(n, heads, generator=g)}.get(which)
        first_needed = max(0, n - new - window + 1) if window else 0
        for i in range(first_needed // page, -(-n // page)):
            table[b, i] = order.pop()
        for p in range((first_needed // page) * page, n):
            k_pages[table[b, p // page], :, p % page] = k[p]
            v_pages[table[b, p // page], :, p % page] = v[p]
        wide = None if gate is None else (gate if which == "all" else gate.repeat_interleave(head_dim, dim=1))
        want = plain_biased_attention(q.double(), k.double(), v.double(), head_dim**-0.5, window or None, slopes, sink, wide)
        q_rows.append(q[n - new :]), want_rows.append(want[n - new :])
        if gate is not None:
            gate_rows.append(gate[n - new :])
        entry_of += [b] * new
        positions += list(range(n - new, n))
    data = dict(new_counts=news, lengths=lengths, entry_of=torch.tensor(entry_of, dtype=torch.int32).cuda(),
                positions=torch.tensor(positions, dtype=torch.int32).cuda())  # fmt: skip
    q_all = torch.cat(q_rows).reshape(-1, heads * head_dim).contiguous().cuda()
    want = torch.cat(want_rows).reshape(-1, heads * head_dim).float()
    out = torch.full_like(q_all, float("nan"))
    assert attention_bf16.tensor_memory_kernel_takes(head_dim, page, window, max(news))
    ops.paged_attention(
        q=q_all, k_pages=k_pages.cuda(), v_pages=v_pages.cuda(), block_table=table.cuda(), ctx=fake_context(data), out=out,
        heads=heads, kv_heads=kv_heads, head_dim=head_dim, scale=head_dim**-0.5, window=window,
        gate=torch.cat(gate_rows).contiguous().cuda() if gate_rows else None,
        slopes=None if slopes is None else slopes.cuda(), sink_values=None if sink is None else sink.cuda(),
    )  # fmt: skip
    torch.cuda.synchronize()
    assert attention_bf16.take_error() == 0
    error = float((out.float().cpu() - want).abs().max()) / float(want.abs().max())
    assert error < 2e-2, f"relative error {error:.3g}"


@pytest.mark.parametrize("rank,rot", [(128, 64), (256, 64), (512, 64), (384, 0)])
@pytest.mark.parametrize("heads,page", [(5, 4), (16, 16), (40, 16)])
@pytest.mark.parametrize("news", [[1, 1, 1, 1], [90, 5, 130, 2], [1, 40, 1, 7], [700, 64, 129, 300]])
@pytest.mark.parametrize("window", [0, 70, 300])
@pytest.mark.parametrize("tensor_memory", [True, False])
def test_tensor_core_attention_over_latent_rows(rank, rot, heads, page, news, window, tensor_memory, monkeypatch):
    """The bfloat16 kernel whose score rows are (token, head) pairs over one cached row per token that is key and,
    in its first elements, value: prompt portions, requests of one token whose keys are split over several CTAs (the
    longest context spans three of them), and both in one step, with a gate per head, over shuffled pages whose free
    places hold large numbers, against float64.  One key of every request stands out for the first head.  Portions of
    64 (token, head) pairs and more over pages of 8 to 64 tokens take the tcgen05 kernel (``tensor_memory``), or the
    ``mma.sync`` kernel when it is switched off."""
    from test_kernels_gpu import fake_context

    from mini_engine_b200.csrc import ops

    monkeypatch.setattr(ops, "LATENT_TENSOR_MEMORY", tensor_memory)
    width = rank + rot
    g = torch.Generator().manual_seed(rank + heads + page + len(news) + window + news[1])
    lengths = [700, 90, 130, 300]
    total_pages = sum(-(-n // page) for n in lengths) + 3
    order = torch.randperm(total_pages, generator=g).tolist()
    pages = torch.full((total_pages, 1, page, width), 1e4).to(torch.bfloat16)
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths) + 1), -1, dtype=torch.int32)
    q_rows, want_rows, gate_rows, entry_of, positions = [], [], [], [], []
    for b, (n, new) in enumerate(zip(lengths, news)):
        q = (0.5 * torch.randn(n, heads, width, generator=g)).to(torch.bfloat16)
        k = torch.randn(n, 1, width, generator=g).to(torch.bfloat16)
        far = max(n - (window or n) + 1, 0) + 2  # a key near the far end of what the last queries see
        k[far, 0] = (k[far, 0].float() + 0.3 * q[n - 1, 0].float()).to(torch.bfloat16)
        gate = torch.rand(n, heads, generator=g)
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
        for p in range(n):
            pages[table[b, p // page], 0, p % page] = k[p, 0]
        want = plain_biased_attention(q.double(), k.double(), k[:, :, :rank].double(), width**-0.5, window or None, gate=gate)
        q_rows.append(q[n - new :]), want_rows.append(want[n - new :]), gate_rows.append(gate[n - new :])
        entry_of += [b] * new
        positions += list(range(n - new, n))
    data = dict(new_counts=news, lengths=lengths, entry_of=torch.tensor(entry_of, dtype=torch.int32).cuda(),
                positions=torch.tensor(positions, dtype=torch.int32).cuda())  # fmt: skip
    q_all = torch.cat(q_rows).reshape(-1, heads * width).contiguous().cuda()
    want = torch.cat(want_rows).reshape(-1, heads * rank).float()
    out = torch.full((q_all.shape[0], heads * rank), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops.latent_attention_supports(width, rank)
    for _ in range(2):  # the second run finds the arrival counters as the first left them
        out.fill_(float("nan"))
        ops.paged_attention(
            q=q_all, k_pages=pages.cuda(), v_pages=None, block_table=table.cuda(), ctx=fake_context(data), out=out, heads=heads,
            kv_heads=1, head_dim=width, scale=width**-0.5, window=window, value_dim=rank, gate=torch.cat(gate_rows).contiguous().cuda(),
        )  # fmt: skip
        torch.cuda.synchronize()
        ops.raise_on_device_error()
        error = float((out.float().cpu() - want).abs().max()) / float(want.abs().max())
        assert error < 2e-2, f"relative error {error:.3g}"


@pytest.mark.parametrize("window", [5, 64, 65, 200, 257])
@pytest.mark.parametrize("offset", ["just_inside", "just_outside", "far", "itself"])
def test_a_key_that_stands_out_at_the_windows_edge_on_tensor_cores(window, offset):
    """As above for the tensor-core kernel over latent rows: the marked value is in the output exactly when its key
    is inside the window, for a query inside a portion and for one that comes alone (split over spans of keys)."""
    from test_kernels_gpu import fake_context

    from mini_engine_b200.csrc import ops

    torch.manual_seed(window)
    T, H, W, R, page = 600, 6, 192, 128, 16
    query = 590
    target = {"just_inside": query - window + 1, "just_outside": query - window, "far": 3, "itself": query}[offset]
    q, k = 0.1 * torch.randn(T, H, W), 0.1 * torch.randn(T, 1, W)
    k[:, :, 0] = 0.0
    q[:, :, 0] = 0.0
    k[target] += 4.0 * q[query, 0] / q[query, 0].norm()
    q[query] = 6.0 * q[query] / q[query].norm(dim=-1, keepdim=True)
    k[target, :, 0] = 100.0
    q, k = q.to(torch.bfloat16), k.to(torch.bfloat16)
    visible = 0 <= query - target < window
    want = plain_biased_attention(q.double(), k.double(), k[:, :, :R].double(), 1.0, window).float()
    generator = torch.Generator().manual_seed(T)
    pages, table = paged(k.float(), page, 3 * (-(-T // page)), generator)
    for new, length in ((1, query + 1), (25, query + 5)):
        rows = list(range(length - new, length))
        data = dict(new_counts=[new], lengths=[length], entry_of=torch.zeros(new, dtype=torch.int32).cuda(),
                    positions=torch.tensor(rows, dtype=torch.int32).cuda())  # fmt: skip
        out = torch.full((new, H * R), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.paged_attention(
            q=q[rows].reshape(new, H * W).contiguous().cuda(), k_pages=pages.to(torch.bfloat16).cuda(), v_pages=None,
            block_table=table.view(1, -1).cuda(), ctx=fake_context(data), out=out, heads=H, kv_heads=1, head_dim=W, scale=1.0,
            window=window, value_dim=R,
        )  # fmt: skip
        torch.cuda.synchronize()
        got = out.float().cpu().view(new, H, R)
        assert (got[rows.index(query), 0, 0] > 50.0) == visible, f"the marked value is {'missing' if visible else 'seen'}"
        assert torch.allclose(got, want[rows], atol=2.0, rtol=2e-2)


@pytest.mark.parametrize("heads,inner,outs,tail,dims", [(3, 128, 200, 16, 8), (2, 512, 128, 0, 0), (5, 64, 520, 64, 64), (1, 192, 8, 8, 0)])
@pytest.mark.parametrize("tokens", [1, 70, 130, 3900])
def test_products_per_head_on_tensor_cores(heads, inner, outs, tail, dims, tokens):
    """The bfloat16 products per head whose inner size is a multiple of 64 run on tensor cores: from partial sums and
    from rounded rows, with a rotated tail, at token counts around the tile of 64, and at one where a CTA walks all
    output chunks of its tile (five heads of 3,900 tokens)."""
    from mini_engine_b200.csrc import ops

    torch.manual_seed(heads + inner + tokens)
    x = torch.randn(2, tokens, heads * (inner + tail))
    weight = torch.randn(heads, inner, outs).to(torch.bfloat16)
    positions = torch.arange(30, 30 + tokens)
    table = None
    if dims:
        freq = torch.tensor([700.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        angle = positions.double().view(-1, 1) * freq
        table = torch.stack((torch.cos(angle), torch.sin(angle)), dim=-1).float()
    rows = x.double().sum(0).view(tokens, heads, inner + tail)
    rounded = rows[..., :inner].to(torch.bfloat16).double()
    want = torch.einsum("thk,hkn->thn", rounded, weight.double())
    if tail:
        rotated = plain.rotate_half(rows[..., inner:], positions, 700.0, dims) if dims else rows[..., inner:]
        want = torch.cat((want, rotated), dim=-1)
    out = torch.full((tokens, heads * (outs + tail)), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.head_product(cuda(x), weight.cuda(), out, tail=tail, cos_sin=cuda(table))
    limit = 1e-2 * float(want.abs().max())
    assert torch.allclose(out.float().cpu().double().view(tokens, heads, -1), want, atol=limit)
    if not tail:
        single = x.sum(0).to(torch.bfloat16)
        out.fill_(float("nan"))
        ops.head_product(single.cuda(), weight.cuda(), out)
        want = torch.einsum("thk,hkn->thn", single.double().view(tokens, heads, inner), weight.double())
        assert torch.allclose(out.float().cpu().double().view(tokens, heads, -1), want, atol=limit)


# ---------------------------------------------------------------------- mechanisms alone: the latent layer


def test_down_projection_finish_norms_rotation_cache_rows_and_gates():
    from mini_engine_b200.csrc import ops

    torch.manual_seed(3)
    T, q_rank, kv_rank, rot_dim, dims, gates, page = 21, 12, 10, 8, 6, 5, 4
    width = q_rank + kv_rank + rot_dim + gates
    down = torch.randn(3, T, width)
    q_w, kv_w = torch.randn(q_rank), torch.randn(kv_rank)
    positions = torch.arange(100, 100 + T)
    freq = torch.tensor([50.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    angle = positions.double().view(-1, 1) * freq
    table = torch.stack((torch.cos(angle), torch.sin(angle)), dim=-1).float()
    slots = torch.randperm(8 * page)[:T].to(torch.int32)
    slots[4] = -1  # a token without a slot writes nothing
    row = down.double().sum(0)
    want_q = plain.rms_norm(row[:, :q_rank], q_w.double(), 1e-4)
    want_c = plain.rms_norm(row[:, q_rank : q_rank + kv_rank], kv_w.double(), 1e-4)
    want_r = plain.rotate_half(row[:, q_rank + kv_rank : q_rank + kv_rank + rot_dim], positions, 50.0, dims)
    want_g = torch.sigmoid(row[:, -gates:])
    for dtype, tolerance in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        pages = torch.full((9, 1, page, kv_rank + rot_dim), 7.0, dtype=dtype, device="cuda")
        q_latent = torch.empty(T, q_rank, dtype=dtype, device="cuda")
        gate = torch.empty(T, gates, dtype=torch.float32, device="cuda")
        ops.latent_down_finish(down=cuda(down), q_rank=q_rank, kv_rank=kv_rank, rot_dim=rot_dim, q_weight=cuda(q_w), kv_weight=cuda(kv_w),
                               eps=1e-4, cos_sin=cuda(table), slot_mapping=cuda(slots), q_latent=q_latent, k_pages=pages, gates=gates, gate_out=gate)  # fmt: skip
        flat = pages.float().cpu().view(-1, kv_rank + rot_dim).double()
        scale = float(want_c.abs().max())
        assert torch.allclose(q_latent.float().cpu().double(), want_q, atol=tolerance * float(want_q.abs().max()))
        assert torch.allclose(gate.cpu().double(), want_g, atol=1e-6)
        written = torch.zeros(flat.shape[0], dtype=torch.bool)
        for t in range(T):
            if slots[t] < 0:
                continue
            written[slots[t]] = True
            assert torch.allclose(flat[slots[t], :kv_rank], want_c[t], atol=tolerance * scale)
            assert torch.allclose(flat[slots[t], kv_rank:], want_r[t], atol=tolerance * float(want_r.abs().max()))
        assert bool((flat[~written] == 7.0).all()), "rows of other slots were touched"


@pytest.mark.parametrize("heads,inner,outs,tail,dims", [(3, 16, 20, 8, 8), (1, 5, 1, 2, 2), (4, 64, 96, 0, 0), (2, 24, 36, 12, 8), (6, 7, 130, 0, 0)])
@pytest.mark.parametrize("tokens", [1, 8, 19])
def test_products_per_head(heads, inner, outs, tail, dims, tokens):
    """out[t, h] = x[t, h] W[h] for every head, from partial sums and from rounded rows, with a rotated tail."""
    from mini_engine_b200.csrc import ops

    torch.manual_seed(heads + inner + tokens)
    x = torch.randn(2, tokens, heads * (inner + tail))
    weight = torch.randn(heads, inner, outs)
    positions = torch.arange(30, 30 + tokens)
    table = None
    if dims:
        freq = torch.tensor([700.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        angle = positions.double().view(-1, 1) * freq
        table = torch.stack((torch.cos(angle), torch.sin(angle)), dim=-1).float()
    for dtype, tolerance in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        w = weight.to(dtype).double()
        rows = x.double().sum(0).view(tokens, heads, inner + tail)
        want = torch.einsum("thk,hkn->thn", rows[..., :inner], w)
        if tail:
            rotated = plain.rotate_half(rows[..., inner:], positions, 700.0, dims) if dims else rows[..., inner:]
            want = torch.cat((want, rotated), dim=-1)
        out = torch.empty(tokens, heads * (outs + tail), dtype=dtype, device="cuda")
        ops.head_product(cuda(x), cuda(weight, dtype), out, tail=tail, cos_sin=cuda(table))
        limit = tolerance * float(want.abs().max())
        assert torch.allclose(out.float().cpu().double().view(tokens, heads, -1), want, atol=limit)
        if not tail:  # rows in the weight's dtype instead of partial sums
            single = x.sum(0).to(dtype)
            ops.head_product(cuda(single), cuda(weight, dtype), out)
            want = torch.einsum("thk,hkn->thn", single.double().view(tokens, heads, inner), w)
            assert torch.allclose(out.float().cpu().double().view(tokens, heads, -1), want, atol=limit)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_one_latent_layer_and_one_biased_layer_against_plain(dtype_name, tmp_path):
    """Models of one layer each, so that nothing else stands between the mixer and the logits."""
    for index, mixer in enumerate((latent(4, 16, 8, 24, 32, 40, 0.25, 30, 1000.0), attention(4, 2, 16, 24, 0.25, 30))):
        kind = "attention" if "kv_heads" in mixer else "latent_attention"
        raw = {"architecture": "Bevadra", "vocab": 40, "width": 32, "norm": {"eps": 1e-5}, "layers": [{"type": kind, "mixer": mixer, "mlp": None}]}
        folder = write_model(tmp_path / str(index), raw, seed=index, scale=20.0)
        requests = {"a": random_ids(1, 90, 40), "b": random_ids(2, 31, 40)}
        replay_and_compare(folder, dtype_name, schedules.changing_portions(requests), requests)


# Sizes that the tensor-core kernels take: attention heads of 128 with a window (tcgen05 for portions of 32 tokens and
# more, the split TMA kernel for single tokens), a reader of its keys with a wider window, latents of 128 and 256 with
# 64 rotated elements (tcgen05 for portions of 64 (token, head) rows and more, split spans for single tokens).
CONFIG_V = {
    "architecture": "Bevadra", "vocab": 72, "width": 128, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
    "layers": [
        {"type": "attention", "mixer": attention(4, 2, 128, 128, 0.09, 70), "mlp": dense(128)},
        {"type": "latent_attention", "mixer": latent(4, 32, 64, 32, 128, 64, 0.1, 50, 10000.0), "mlp": dense(64)},
        {"type": "attention", "mixer": attention(4, 2, 128, 128, 0.08, 150, kv_from=0), "mlp": None},
        {"type": "latent_attention", "mixer": latent(5, 64, 64, 48, 256, 128, 0.09, 200, 500.0, dims=32), "mlp": dense(128)},
    ],
}  # fmt: skip


@pytest.mark.parametrize("schedule", ["whole", "tail_one_by_one", "changing_portions", "mixed"])
def test_sizes_that_the_tensor_core_kernels_take(schedule, tmp_path_factory):
    """A model whose bfloat16 steps run the tcgen05 and split kernels of both mixers, against the plain model, with
    prompts longer than every window and than two blocks of 128 rows."""
    folder = write_model(tmp_path_factory.mktemp("bevadra_V"), CONFIG_V, scale=6.0)
    requests = {f"r{i}": random_ids(700 + i, n, CONFIG_V["vocab"]) for i, n in enumerate([300, 64, 161, 230, 33])}
    maker = {"whole": schedules.whole, "changing_portions": schedules.changing_portions, "mixed": schedules.mixed,
             "tail_one_by_one": lambda r: schedules.tail_one_by_one(r, 40)}[schedule]  # fmt: skip
    replay_and_compare(folder, "bfloat16", maker(requests), requests)


# ---------------------------------------------------------------------- the engine's own entry point


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["S", "T"])
def test_greedy_generation_through_the_engine(folders, dtype_name, name):
    """`LLMEngine.generate`: the scheduler, portions under a 48-token budget, captured decode steps, prefix hits.
    Every generated token is checked teacher-forced: its plain logit lies within the tolerance of the largest one
    at its position."""
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = folders[name]
    weights, config = load_plain(folder)
    prompts = [random_ids(40 + i, n, config["vocab"]) for i, n in enumerate((19, 70, 3, 41, 100))]
    engine = LLMEngine.from_pretrained(
        folder, EngineConfig(block_size=16, num_blocks=64, max_model_len=256, max_num_seqs=3, max_num_batched_tokens=48,
                             dtype=DTYPES[dtype_name])  # fmt: skip
    )
    got = engine.generate(prompts, SamplingParams(max_tokens=24, ignore_eos=True))
    assert engine.stats.graph_steps > 0

    def check(prompts, generated):
        for prompt, tokens in zip(prompts, generated):
            assert len(tokens) == 24
            logits = plain.forward(config, weights, (prompt + tokens)[:-1]).float()
            slack = 2 * TOLERANCE[dtype_name] * float(logits.abs().max())
            for i, token in enumerate(tokens):
                row = logits[len(prompt) - 1 + i]
                assert float(row.max() - row[token]) <= slack, f"token {i} of a {len(prompt)}-token prompt"

    check(prompts, got)
    # pages of finished requests, and the prefixes that are still cached, serve new requests
    again = engine.generate(prompts[:2], SamplingParams(max_tokens=24, ignore_eos=True))
    check(prompts[:2], again)
    if dtype_name == "float32":
        assert again == got[:2]


def test_the_command_line(folders, capsys):
    """`python -m mini_engine_b200.cli.generate` on a folder of this design: greedy output equals the engine's, and a
    run with temperature draws tokens of the vocabulary through the device sampler."""
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_engine_b200.cli import generate

    folder = str(folders["S"])
    prompts = [random_ids(70 + i, n, CONFIG_S["vocab"]) for i, n in enumerate((12, 30))]
    ids = ";".join(",".join(map(str, p)) for p in prompts)
    common = ["--model", folder, "--dtype", "fp32", "--max-tokens", "6", "--ignore-eos", "--num-blocks", "32", "--max-model-len", "128",
              "--max-num-seqs", "2", "--prompt-ids", ids]  # fmt: skip
    assert generate.main(common) == 0
    greedy = capsys.readouterr().out
    engine = LLMEngine.from_pretrained(folder, EngineConfig(block_size=16, num_blocks=32, max_model_len=128, max_num_seqs=2, dtype=torch.float32))
    want = engine.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    for prompt, tokens in zip(prompts, want):
        assert f"prompt ({len(prompt)} tokens) -> {tokens}" in greedy
    assert generate.main(common + ["--temperature", "0.8", "--seed", "3"]) == 0
    drawn = capsys.readouterr().out.splitlines()[:2]
    for line, prompt in zip(drawn, prompts):
        tokens = json.loads(line.split("-> ")[1])
        assert line.startswith(f"prompt ({len(prompt)} tokens)") and len(tokens) == 6 and all(0 <= t < CONFIG_S["vocab"] for t in tokens)


def test_preempted_requests_are_computed_again(folders):
    """A pool so small that running requests are preempted: their pages go back, they are computed again, and the
    tokens are those of a run with room for everyone."""
    from mini_engine_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = folders["T"]
    prompts = [random_ids(90 + i, n, CONFIG_T["vocab"]) for i, n in enumerate((40, 33, 25, 47))]
    params = SamplingParams(max_tokens=30, ignore_eos=True)
    roomy = LLMEngine.from_pretrained(folder, EngineConfig(block_size=16, num_blocks=64, max_model_len=128, max_num_seqs=4, dtype=torch.float32))
    want = roomy.generate(prompts, params)
    tight = LLMEngine.from_pretrained(folder, EngineConfig(block_size=16, num_blocks=11, max_model_len=128, max_num_seqs=4, dtype=torch.float32))
    got = tight.generate(prompts, params)
    assert tight.scheduler.num_preemptions > 0
    assert got == want
