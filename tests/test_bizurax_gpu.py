"""The Bizurax design through the framework against the plain implementation of ``plain_bizurax.py``: each mechanism
alone, whole prompts against portions and token-by-token decoding, mixed batches with pages and state slots that are
used again, far keys that stand out, long decoding, several sizes, and greedy generation through the engine's entry
point."""

from __future__ import annotations

import json
import math
import random
from pathlib import Path

import pytest
import torch

import plain_bizurax as plain
import schedules
from conftest import note_error

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# Largest |engine - plain| relative to the request's largest |logit|.
TOLERANCE = {"float32": 3e-5, "bfloat16": 6e-2}
# A router's choice that was won by less than this (in logits) may fall the other way when activations are rounded to
# bfloat16, and everything behind it follows the other choice.  In bfloat16 the plain implementation is therefore told
# what the engine chose and takes that where its own decision was this close (a differing choice on a clear decision
# fails the comparison); float32 is compared without any of this.
CLOSE_CALL = 0.2


def rot(base, dims, factor=None):
    out = {"base": base, "dims": dims}
    if factor:
        out["scaling"] = {"factor": factor}
    return out


def attention(heads, kv_heads, dim, vdim, scale, softcap, rotation):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotation}
    if softcap:
        out["softcap"] = softcap
    return out


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot(base, rot_dim)}


def retention(heads, dim, vdim, decay, rotation):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": rotation}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


# Three streams; a loop over two layers in the middle; all three mixers; heads rotated in part and with scaled
# frequencies; value heads wider and narrower than key heads; groups of three heads; a layer without feed-forward;
# routed units with and without a shared one; an attention layer without a cap.
CONFIG_S = {
    "architecture": "Bizurax", "vocab": 90, "width": 48, "norm": {"eps": 2e-5}, "residual_mult": 0.7, "streams": 3,
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        {"type": "latent_attention", "mixer": latent(3, 16, 8, 24, 20, 0.2, 300.0), "mlp": dense(40)},
        {"type": "retention", "mixer": retention(3, 16, 24, [0.9, 0.99, 1.0], rot(1000.0, 8)), "mlp": moe(5, 2, 16, 24)},
        {"type": "attention", "mixer": attention(6, 2, 16, 24, 0.5, 3.0, rot(500.0, 12, 2.0)), "mlp": None},
        {"type": "attention", "mixer": attention(2, 2, 24, 8, 0.3, None, rot(10000.0, 24)), "mlp": moe(4, 1, 24)},
        {"type": "retention", "mixer": retention(1, 24, 8, [0.95], rot(100.0, 24, 3.0)), "mlp": dense(16)},
    ],
}  # fmt: skip
# Widths that the tensor-core products take, heads of 64 and 128, the whole model inside the loop, two streams.
CONFIG_T = {
    "architecture": "Bizurax", "vocab": 64, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "streams": 2,
    "loop": {"start": 0, "stop": 3, "times": 2},
    "layers": [
        {"type": "attention", "mixer": attention(4, 2, 64, 64, 0.125, 30.0, rot(500000.0, 64, 8.0)), "mlp": dense(64)},
        {"type": "retention", "mixer": retention(2, 64, 64, [0.96875, 0.998], rot(2e5, 64)), "mlp": moe(8, 3, 64, 128)},
        {"type": "latent_attention", "mixer": latent(4, 32, 32, 32, 64, 0.15, 40000.0), "mlp": moe(8, 2, 32, 64)},
    ],
}  # fmt: skip
# Sizes that no fast path takes: a width that is no multiple of 8, odd head widths, one head, one stream, one routed
# unit, as many choices as units, a rotation of two elements, a rank of one, a loop that runs once, no multiplier.
CONFIG_U = {
    "architecture": "Bizurax", "vocab": 51, "width": 36, "norm": {"eps": 1e-4}, "streams": 1,
    "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [
        {"type": "attention", "mixer": attention(1, 1, 10, 6, 0.6, 1.5, rot(30.0, 2)), "mlp": moe(1, 1, 9)},
        {"type": "latent_attention", "mixer": latent(1, 5, 2, 7, 1, 0.5, 20.0), "mlp": dense(17)},
        {"type": "retention", "mixer": retention(3, 6, 5, [0.5, 0.75, 0.999], rot(50.0, 4)), "mlp": moe(3, 3, 7, 5)},
        {"type": "attention", "mixer": attention(3, 1, 14, 20, 0.4, 50.0, rot(1000.0, 6, 1.5)), "mlp": None},
    ],
}  # fmt: skip
# One plain residual (no streams), no loop: the pre-norm sum with the model's multiplier.
CONFIG_P = {
    "architecture": "Bizurax", "vocab": 70, "width": 40, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
    "layers": [
        {"type": "retention", "mixer": retention(2, 8, 16, [0.97, 0.9], rot(200.0, 8)), "mlp": dense(24)},
        {"type": "attention", "mixer": attention(4, 1, 8, 8, 1.0, 10.0, rot(200.0, 8)), "mlp": None},
        {"type": "latent_attention", "mixer": latent(2, 8, 4, 8, 12, 0.3, 100.0), "mlp": moe(6, 2, 8, 8)},
    ],
}  # fmt: skip
CONFIGS = {"S": CONFIG_S, "T": CONFIG_T, "U": CONFIG_U, "P": CONFIG_P}
LENGTHS = {"S": [70, 45, 133, 9, 97, 33, 1, 2], "T": [150, 64, 17, 81, 49, 130], "U": [40, 3, 77, 18, 1, 60], "P": [50, 2, 90, 31, 1]}


def random_ids(seed, count, vocab):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]


def write_model(folder, raw, seed=31, scale=8.0):
    from mini_engine_b200.config import BizuraxConfig
    from mini_engine_b200.weights import write_random_model

    write_random_model(folder, BizuraxConfig.from_dict(raw), seed=seed, dtype=torch.bfloat16, scale=scale)
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_model(tmp_path_factory.mktemp(f"bizurax_{name}"), raw) for name, raw in CONFIGS.items()}


def load_plain(folder):
    from safetensors.torch import load_file

    weights = {k: v.to(torch.float64) for k, v in load_file(str(Path(folder) / "model.safetensors")).items()}
    return weights, json.loads((Path(folder) / "config.json").read_text())


def routed_runs(config):
    """The layer runs (in running order) whose feed-forward is routed."""
    return [run for run, index in enumerate(plain.layer_order(config)) if (config["layers"][index].get("mlp") or {}).get("kind") == "moe"]


def expected_logits(folder, requests, routing=None, nudge=0.0):
    """Plain logits per request.  ``routing`` (request -> layer run -> [T, top]) is the engine's choice, followed where
    the plain decision was a close call.  ``nudge``: the relative size of a random change of every embedding element."""
    weights, config = load_plain(folder)
    if nudge:
        noise = torch.randn(weights["embed"].shape, generator=torch.Generator().manual_seed(7), dtype=torch.float64)
        weights = dict(weights, embed=weights["embed"] * (1.0 + nudge * noise))
    out = {}
    for name, toks in requests.items():
        follow = None if routing is None else routing.get(name)
        out[name] = plain.forward(config, weights, toks, follow=follow, close=CLOSE_CALL).float()
    return out


def replay(folder, dtype_name, steps, block_size=16, max_tokens=None, max_live=4, max_step_tokens=512, routing=None):
    """``routing`` (a dict) is filled with what the routed feed-forwards chose: request -> layer run -> [T, top]."""
    from mini_engine_b200.engine.replay import Replayer
    from mini_engine_b200.parts import moe as moe_module

    replayer = Replayer(folder, DTYPES[dtype_name], max_tokens or schedules.peak_live_tokens(steps), block_size,
                        max_step_tokens=max_step_tokens, max_live=max_live)  # fmt: skip
    runs = routed_runs(json.loads((Path(folder) / "config.json").read_text()))
    calls: list = []
    original = moe_module.RoutedExperts._forward_routed

    def recording(self, h, ctx, chosen, chosen_weight, weights):
        calls.append(chosen.clone())
        return original(self, h, ctx, chosen, chosen_weight, weights)

    outputs = {}
    moe_module.RoutedExperts._forward_routed = recording
    try:
        for record in steps:
            calls.clear()
            logits = replayer.step(record)
            if logits is not None:
                outputs[record["step"]] = logits.clone()
            if routing is not None and record["entries"]:
                assert len(calls) == len(runs)
                first = 0
                for item in record["entries"]:
                    count = len(item["tokens"])
                    for run, chosen in zip(runs, calls):
                        held = routing.setdefault(item["id"], {}).setdefault(run, [])
                        held.append(chosen[first : first + count].cpu())
                    first += count
    finally:
        moe_module.RoutedExperts._forward_routed = original
    if routing is not None:
        for per_run in routing.values():
            for run in per_run:
                per_run[run] = torch.cat(per_run[run]) if isinstance(per_run[run], list) else per_run[run]
    replayer.manager.check_invariants([])
    assert all(pool.num_free == pool.num_pages for pool in replayer.manager.pools), "pages were lost"
    return schedules.collect(steps, outputs)


def compare(got, expected, requests, dtype_name, nudged=None):
    """``nudged``: the plain logits of a model whose embedding was changed by about a bfloat16 rounding (a relative 2^-10, normally distributed).  Where they
    leave the plain logits by a quarter of the tolerance, the position hangs on a close call of the design itself (the
    sign of a retention head's lone product in front of its unit norm, say) and says nothing about the engine; such
    positions must be few, and float32 checks them all."""
    worst, skipped, total = 0.0, 0, 0
    for name, toks in requests.items():
        assert sorted(got[name]) == list(range(len(toks))), f"{name}: positions missing"
        scale = float(expected[name].abs().max())
        for position, row in got[name].items():
            total += 1
            if nudged is not None and float((nudged[name][position] - expected[name][position]).abs().max()) / scale > TOLERANCE[dtype_name] / 4:
                skipped += 1
                continue
            error = float((row - expected[name][position]).abs().max()) / scale
            worst = max(worst, error)
            assert error <= TOLERANCE[dtype_name], f"{name} position {position}: relative error {error:.3g}"
    assert skipped <= max(2, 0.05 * total), f"{skipped} of {total} positions hang on close calls"
    note_error("bizurax " + dtype_name, worst)


def replay_and_compare(folder, dtype_name, steps, requests, **options):
    routing = {} if dtype_name == "bfloat16" else None
    got = replay(folder, dtype_name, steps, routing=routing, **options)
    nudged = expected_logits(folder, requests, routing, nudge=2.0**-10) if dtype_name == "bfloat16" else None
    compare(got, expected_logits(folder, requests, routing), requests, dtype_name, nudged)


def requests_for(name):
    return {f"r{i}": random_ids(500 + i, n, CONFIGS[name]["vocab"]) for i, n in enumerate(LENGTHS[name])}


# --------------------------------------------------------------- whole models, every way of cutting


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["S", "T", "U", "P"])
@pytest.mark.parametrize("schedule", ["whole", "tail_one_by_one", "changing_portions", "mixed"])
def test_schedules_match_plain(name, dtype_name, schedule, folders):
    """Whole prompts (requests of one and two tokens among them); the last 32 tokens one by one; portions down to two
    tokens; up to four live requests whose pages and state slots are handed out again."""
    requests = requests_for(name)
    steps = getattr(schedules, schedule)(requests)
    replay_and_compare(folders[name], dtype_name, steps, requests)


@pytest.mark.parametrize("block_size", [4, 16, 32])
def test_float32_hardly_depends_on_the_cut_or_the_batch(folders, block_size, monkeypatch):
    """In float32 every kernel's sums for a token depend on that token's position alone, except that retention runs long
    portions in chunks whose sums are ordered by the chunk's place in the portion: portions, single tokens, mixed
    batches and other page sizes give the whole prompt's logits up to that rounding, and its very bits when every
    portion walks token by token."""
    from mini_engine_b200.parts import linear_attention

    requests = {name: toks for name, toks in list(requests_for("S").items())[:5]}
    for chunked in (True, False):
        if not chunked:
            monkeypatch.setattr(linear_attention, "CHUNKED_MIN_TOKENS", 1 << 30)
        whole = replay(folders["S"], "float32", schedules.whole(requests), block_size)
        for maker in (schedules.changing_portions, schedules.mixed, lambda r: schedules.tail_one_by_one(r, 40)):
            cut = replay(folders["S"], "float32", maker(requests), block_size)
            for name, toks in requests.items():
                for position in range(len(toks)):
                    a, b = whole[name][position], cut[name][position]
                    if chunked:
                        assert float((a - b).abs().max()) <= 1e-5 * float(a.abs().max()), f"{name} position {position}"
                    else:
                        assert torch.equal(a, b), f"{name} position {position}"


def test_long_decoding(folders):
    """Three prompt tokens, then 200 tokens one by one: the state is carried through 200 steps, the caches grow page by page."""
    for name in ("S", "T"):
        requests = {"long": random_ids(77, 203, CONFIGS[name]["vocab"])}
        steps = schedules.tail_one_by_one(requests, tail=200)
        for dtype_name in ("float32", "bfloat16"):
            replay_and_compare(folders[name], dtype_name, steps, requests)


def test_pages_and_slots_that_are_used_again_hold_nothing_of_their_past(folders):
    """A pool of four pages and one state slot: the second request gets the first one's pages and its slot, and must
    see neither the keys nor the state that they held."""
    from mini_engine_b200.engine.replay import Replayer

    a, b = random_ids(5, 60, CONFIG_S["vocab"]), random_ids(6, 37, CONFIG_S["vocab"])
    replayer = Replayer(folders["S"], torch.float32, 64, 16, max_live=1)
    first = replayer.step({"step": 0, "entries": [{"id": "a", "tokens": a, "want": [59]}], "end": ["a"]})
    assert replayer.step({"step": 1, "entries": [{"id": "b", "tokens": b[:20], "want": []}], "end": []}) is None
    second = replayer.step({"step": 2, "entries": [{"id": "b", "tokens": b[20:], "want": [16]}], "end": ["b"]})
    alone = Replayer(folders["S"], torch.float32, 64, 16).step({"step": 0, "entries": [{"id": "b", "tokens": b, "want": [36]}], "end": ["b"]})
    assert torch.allclose(second, alone, atol=1e-5 * float(alone.abs().max())) and not torch.allclose(first, alone, atol=1e-2)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_the_replay_program_itself(folders, dtype_name, tmp_path):
    """`bin/trace_run` as a process on a model folder of this design: mixed steps in, `done` lines and logit files out."""
    import subprocess
    import sys

    import numpy as np
    from conftest import ROOT

    requests = requests_for("P")
    steps = schedules.mixed(requests)
    out = tmp_path / "out"
    feed = "".join(json.dumps(record) + "\n" for record in steps)
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders["P"]), "--dtype", dtype_name,
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
            outputs[record["step"]] = torch.from_numpy(data.reshape(wanted, CONFIG_P["vocab"]).copy())
    got = schedules.collect(steps, outputs)
    if dtype_name == "float32":
        compare(got, expected_logits(folders["P"], requests), requests, dtype_name)
    else:  # the process keeps its routing to itself: against the same steps in this process, bit for bit
        here = replay(folders["P"], dtype_name, steps)
        for name, toks in requests.items():
            for position in range(len(toks)):
                assert torch.equal(got[name][position], here[name][position])


def test_the_streams_after_every_layer_run(folders):
    """The sum of the residual streams behind each layer run (a looped layer counts each time), with the update that
    the last sublayer's output is still owed, against the plain layers, in float32."""
    from mini_engine_b200.csrc import ops
    from mini_engine_b200.engine.replay import Replayer
    from mini_engine_b200.parts import block as block_module

    weights, config = load_plain(folders["S"])
    toks = random_ids(9, 50, config["vocab"])
    _, want = plain.forward(config, weights, toks, return_layers=True)
    seen = []
    original = block_module.HyperConnectionBlock.forward

    def recording(self, state, ctx, cache):
        original(self, state, ctx, cache)
        total = torch.empty_like(state.x)
        mix, share, mult = state.stream_update
        ops.hyper_sum(streams=state.streams, seed=state.x if state.streams_unwritten else None, pending=state.pending,
                      mix=mix, share=share, mult=mult, out=total)  # fmt: skip
        seen.append(total)

    block_module.HyperConnectionBlock.forward = recording
    try:
        Replayer(folders["S"], torch.float32, 64).step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": ["a"]})
    finally:
        block_module.HyperConnectionBlock.forward = original
    assert len(seen) == len(plain.layer_order(config)) == 7
    for index, got in enumerate(seen):
        assert torch.allclose(got.cpu(), want[index].float(), atol=2e-5 * float(want[index].abs().max())), f"layer run {index}"


# ---------------------------------------------------------------------- mechanisms alone: small kernels


def cuda(t, dtype=None):
    return None if t is None else t.to(device="cuda", dtype=dtype or t.dtype).contiguous()


class Context:
    """What the kernels' bindings read of a step: one entry per request."""

    def __init__(self, counts, starts, slots):
        self.num_entries = len(counts)
        cu = [0]
        for n in counts:
            cu.append(cu[-1] + n)
        self.cu_tokens = torch.tensor(cu, dtype=torch.int32, device="cuda")
        self.state_slots = torch.tensor(slots, dtype=torch.int32, device="cuda")
        self.fresh = torch.tensor([1 if s == 0 else 0 for s in starts], dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("count", [1, 2, 4, 8])
@pytest.mark.parametrize("hidden", [36, 48, 1000])
@pytest.mark.parametrize("splits", [1, 3])
def test_hyper_connection_step(count, hidden, splits):
    """The update of all streams from the old ones, their write-back, the weighted read and its norm; then the same
    with streams that have not been written yet (all equal the seed rows), with rows picked, and without an update."""
    from mini_engine_b200.csrc import ops

    g = torch.Generator().manual_seed(count * 1000 + hidden)
    tokens, mult, eps = 7, 0.6, 1e-5
    streams = torch.randn(count, tokens, hidden, generator=g, dtype=torch.float64)
    pending = torch.randn(splits, tokens, hidden, generator=g, dtype=torch.float64)
    mix = torch.randn(count, count, generator=g, dtype=torch.float64)
    share, read = torch.randn(count, generator=g, dtype=torch.float64), torch.randn(count, generator=g, dtype=torch.float64)
    weight = 1 + 0.1 * torch.randn(hidden, generator=g, dtype=torch.float64)

    def plain_step(old, y, read_weights):
        fresh = old if y is None else torch.einsum("sr,stw->rtw", mix, old) + mult * share.view(-1, 1, 1) * y
        u = fresh.sum(0) if read_weights is None else torch.einsum("s,stw->tw", read_weights, fresh)
        return fresh, plain.rms_norm(u, weight, eps)

    for out_dtype, tolerance in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        held = cuda(streams, torch.float32)
        out = torch.empty(tokens, hidden, dtype=out_dtype, device="cuda")
        ops.hyper_step(streams=held, seed=None, pending=cuda(pending, torch.float32), mix=cuda(mix, torch.float32),
                       share=cuda(share, torch.float32), mult=mult, read=cuda(read, torch.float32), weight=cuda(weight, torch.float32),
                       eps=eps, out=out)  # fmt: skip
        fresh, normed = plain_step(streams, pending.sum(0), read)
        assert torch.allclose(held.cpu().double(), fresh, atol=1e-5 * float(fresh.abs().max()))
        assert torch.allclose(out.cpu().double(), normed, atol=tolerance * float(normed.abs().max()))
    # streams that were never written: every one is the seed; rows picked: nothing is written back
    seed = streams[0]
    held = torch.full((count, tokens, hidden), float("nan"), dtype=torch.float32, device="cuda")
    out = torch.empty(tokens, hidden, dtype=torch.float32, device="cuda")
    common = dict(mix=cuda(mix, torch.float32), share=cuda(share, torch.float32), mult=mult, weight=cuda(weight, torch.float32), eps=eps)
    ops.hyper_step(streams=held, seed=cuda(seed, torch.float32), pending=None, read=cuda(read, torch.float32), out=out, **common)
    assert torch.isnan(held).all()  # no update is owed: the streams stay unwritten
    assert torch.allclose(out.cpu().double(), plain_step(seed.expand(count, -1, -1), None, read)[1], atol=1e-5 * 4)
    ops.hyper_step(streams=held, seed=cuda(seed, torch.float32), pending=cuda(pending, torch.float32), read=cuda(read, torch.float32), out=out, **common)
    fresh, normed = plain_step(seed.expand(count, -1, -1), pending.sum(0), read)
    assert torch.allclose(held.cpu().double(), fresh, atol=1e-5 * float(fresh.abs().max()))
    assert torch.allclose(out.cpu().double(), normed, atol=1e-5 * float(normed.abs().max()))
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
    before = held.clone()
    picked = torch.empty(3, hidden, dtype=torch.float32, device="cuda")
    ops.hyper_step(streams=held, seed=None, pending=cuda(pending, torch.float32), read=None, out=picked, rows=rows, **common)
    assert torch.equal(held, before)
    _, normed = plain_step(fresh, pending.sum(0), None)
    assert torch.allclose(picked.cpu().double(), normed[[5, 0, 5]], atol=1e-5 * float(normed.abs().max()))


@pytest.mark.parametrize("width", [17, 64])
def test_squared_relu_on_partial_sums(width):
    from mini_engine_b200.csrc import ops

    g = torch.Generator().manual_seed(width)
    sums = torch.randn(3, 9, width, generator=g)
    for dtype, tolerance in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        out = torch.empty(9, width, dtype=dtype, device="cuda")
        ops.activation(cuda(sums), out, "relu_squared")
        want = torch.relu(sums.double().sum(0)) ** 2
        assert torch.allclose(out.cpu().double(), want, atol=tolerance * float(want.abs().max()))
        assert (out.cpu()[sums.sum(0) < 0] == 0).all()


@pytest.mark.parametrize("units,top", [(12, 3), (5, 5), (7, 1), (1, 1), (64, 6)])
def test_router_with_a_bias_and_a_softmax_over_the_chosen(units, top):
    from mini_engine_b200.csrc import ops

    g = torch.Generator().manual_seed(units)
    tokens, hidden = 33, 40
    h = torch.randn(tokens, hidden, generator=g)
    w = {"router": torch.randn(units, hidden, generator=g).double(), "router.b": 3 * torch.randn(units, generator=g).double()}
    want_units, want_weights = plain.route(h.double(), w, "", top)
    dense_map = torch.empty(tokens, units, dtype=torch.float32, device="cuda")
    chosen = torch.empty(tokens, top, dtype=torch.int32, device="cuda")
    chosen_weight = torch.empty(tokens, top, dtype=torch.float32, device="cuda")
    ops.route(h=cuda(h), router=cuda(w["router"], torch.float32), weights=dense_map, chosen=chosen, chosen_weight=chosen_weight,
              top=top, group_count=1, group_keep=1, weight_scale=1.0, bias=cuda(w["router.b"], torch.float32), scoring="softmax_chosen")  # fmt: skip
    assert torch.equal(chosen.cpu().long(), want_units)  # the largest logit first
    assert torch.allclose(chosen_weight.cpu().double(), want_weights, atol=1e-5)
    assert torch.allclose(chosen_weight.sum(-1).cpu(), torch.ones(tokens), atol=1e-5)
    scattered = torch.zeros(tokens, units, dtype=torch.float64).scatter_(1, want_units, want_weights)
    assert torch.allclose(dense_map.cpu().double(), scattered, atol=1e-5)
    # without the bias other units win: the bias is part of the decision
    if units > top:
        ops.route(h=cuda(h), router=cuda(w["router"], torch.float32), weights=dense_map, chosen=chosen, chosen_weight=chosen_weight,
                  top=top, group_count=1, group_keep=1, weight_scale=1.0, scoring="softmax_chosen")  # fmt: skip
        assert not torch.equal(chosen.cpu().long(), want_units)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,dims", [(4, 2, 16, 8, 16), (6, 3, 40, 72, 12), (3, 1, 10, 33, 2), (2, 2, 128, 128, 64), (1, 1, 4, 1, 4)])
@pytest.mark.parametrize("unit", [True, False])
def test_bias_rotation_unit_norm_and_cache_write(heads, kv_heads, dim, vdim, dims, unit):
    """q and k: partial sums + bias, rotation of the first ``dims`` elements, then the root mean square over the whole
    head; v: partial sums + bias.  The norm stands behind the rotation: with a rotation on a part of the head and a
    norm in front of it the result would differ where eps matters, so eps is large here."""
    from mini_engine_b200.csrc import ops

    g = torch.Generator().manual_seed(dim)
    tokens, page, eps, rotation = 21, 4, 0.3, {"base": 77.0, "dims": dims, "scaling": {"factor": 2.0}}
    width = (heads + kv_heads) * dim + kv_heads * vdim
    sums = torch.randn(2, tokens, width, generator=g, dtype=torch.float64)
    bias = torch.randn(width, generator=g, dtype=torch.float64)
    positions = torch.tensor(random.Random(1).sample(range(500), tokens))
    row = sums.sum(0) + bias
    q, k, v = row[:, : heads * dim], row[:, heads * dim : (heads + kv_heads) * dim], row[:, (heads + kv_heads) * dim :]
    q = plain.rotate(q.view(tokens, heads, dim), positions, rotation, False)
    k = plain.rotate(k.view(tokens, kv_heads, dim), positions, rotation, False)
    if unit:
        q, k = plain.rms_norm(q, None, eps), plain.rms_norm(k, None, eps)
    angle = positions.double().view(-1, 1) * plain.frequencies(rotation, sums)
    table = torch.stack((torch.cos(angle), torch.sin(angle)), dim=-1)
    slots = torch.tensor(random.Random(2).sample(range(8 * page), tokens), dtype=torch.int32)
    for dtype, tolerance in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        q_out = torch.empty(tokens, heads * dim, dtype=dtype, device="cuda")
        k_pages = torch.zeros(9, kv_heads, page, dim, dtype=dtype, device="cuda")
        v_pages = torch.zeros(9, kv_heads, page, vdim, dtype=dtype, device="cuda")
        ops.qkv_rope_unit_store(
            qkv=cuda(sums, torch.float32), heads=heads, kv_heads=kv_heads, head_dim=dim, value_dim=vdim, bias=cuda(bias, torch.float32),
            cos_sin=cuda(table, torch.float32), unit_norm_eps=eps if unit else None, q_out=q_out, page_size=page,
            slot_mapping=cuda(slots), k_pages=k_pages, v_pages=v_pages,
        )  # fmt: skip
        assert torch.allclose(q_out.cpu().double().view(tokens, heads, dim), q, atol=tolerance * float(q.abs().max()))
        got_k = k_pages.cpu().double().permute(0, 2, 1, 3).reshape(-1, kv_heads, dim)[slots.long()]
        got_v = v_pages.cpu().double().permute(0, 2, 1, 3).reshape(-1, kv_heads, vdim)[slots.long()]
        assert torch.allclose(got_k, k, atol=tolerance * float(k.abs().max()))
        assert torch.allclose(got_v, v.view(tokens, kv_heads, vdim), atol=tolerance * float(v.abs().max()))


def paged(rows, page_size, pages_total, generator):
    """Scatter ``rows [T, heads, d]`` of one request over pages in a shuffled order; returns the page array
    ``[pages_total + 1, heads, page_size, d]`` and the request's block table."""
    tokens, heads, d = rows.shape
    need = -(-tokens // page_size)
    order = torch.randperm(pages_total, generator=generator)[:need]
    pages = torch.zeros(pages_total + 1, heads, page_size, d, dtype=rows.dtype)
    for t in range(tokens):
        pages[order[t // page_size], :, t % page_size] = rows[t]
    return pages, order.to(torch.int32)


def plain_capped_attention(q, k, v, scale, cap, sink):
    """q [T, H, d] (the last T positions of the request), k [N, G, d], v [N, G, dv], all float64."""
    tokens, heads, _ = q.shape
    total, groups = k.shape[0], k.shape[1]
    kk, vv = k.repeat_interleave(heads // groups, dim=1), v.repeat_interleave(heads // groups, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if cap:
        scores = cap * torch.tanh(scores / cap)
    i = torch.arange(total - tokens, total).view(-1, 1)
    seen = torch.arange(total).view(1, -1) <= i
    weights = plain.softmax_with_extra(scores, seen, sink)
    return torch.einsum("hij,jhd->ihd", weights, vv)


def run_attention(q, k, v, scale, cap, sink, dtype, page_size=16):
    from mini_engine_b200.csrc import ops

    g = torch.Generator().manual_seed(3)
    tokens, heads, dim = q.shape
    total, groups, vdim = k.shape[0], k.shape[1], v.shape[2]
    k_pages, table = paged(k, page_size, 2 * (-(-total // page_size)) + 1, g)
    v_pages, _ = paged(v, page_size, 2 * (-(-total // page_size)) + 1, torch.Generator().manual_seed(3))
    out = torch.empty(tokens, heads * vdim, dtype=dtype, device="cuda")
    ops.paged_attention_generic(
        cuda(q.reshape(tokens, heads * dim), dtype), cuda(k_pages, dtype), cuda(v_pages, dtype), cuda(table.view(1, -1)),
        torch.zeros(tokens, dtype=torch.int32, device="cuda"), torch.arange(total - tokens, total, dtype=torch.int32, device="cuda"),
        out, heads, groups, dim, scale, 0, value_dim=vdim, sink_values=cuda(sink, torch.float32), softcap=cap or 0.0,
    )  # fmt: skip
    return out.cpu().double().view(tokens, heads, vdim)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 16, 8), (6, 3, 40, 72), (3, 1, 10, 33), (1, 1, 4, 1)])
@pytest.mark.parametrize("cap", [None, 2.0, 30.0])
def test_attention_with_capped_scores_and_a_sink_alone(heads, kv_heads, dim, vdim, cap):
    g = torch.Generator().manual_seed(heads * 100 + dim)
    total, tokens = 75, 30
    q = torch.randn(tokens, heads, dim, generator=g, dtype=torch.float64)
    k = torch.randn(total, kv_heads, dim, generator=g, dtype=torch.float64)
    v = torch.randn(total, kv_heads, vdim, generator=g, dtype=torch.float64)
    sink = torch.randn(heads, generator=g, dtype=torch.float64) * 2
    want = plain_capped_attention(q, k, v, 0.7, cap, sink)
    got = run_attention(q, k, v, 0.7, cap, sink, torch.float32)
    assert torch.allclose(got, want, atol=2e-5 * float(want.abs().max()))
    if cap == 2.0:  # the cap matters here: without it the result is another
        assert not torch.allclose(got, plain_capped_attention(q, k, v, 0.7, None, sink), atol=1e-3)
    # the sink only takes weight away: the outputs are those of the plain softmax, shrunk
    no_sink = plain_capped_attention(q, k, v, 0.7, cap, torch.full((heads,), -1e9, dtype=torch.float64))
    assert (want.norm(dim=-1) < no_sink.norm(dim=-1) + 1e-9).all()


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("where", ["first", "page_border", "far", "last"])
def test_a_far_key_that_stands_out(where, dtype_name):
    """Hundreds of keys with small scores and one whose score stands out (its key is the query's direction, scaled):
    the output is that key's value, wherever it lies (the sequence's first token, a page's last slot, far back, the
    query itself); the cap bounds its score, so that the sink and the others keep a known share."""
    g = torch.Generator().manual_seed(11)
    total, dim, vdim, cap, scale = 600, 32, 16, 12.0, 1.0
    place = {"first": 0, "page_border": 15 + 16 * 20, "far": 37, "last": total - 1}[where]
    q = torch.randn(1, 2, dim, generator=g, dtype=torch.float64)
    k = 0.05 * torch.randn(total, 1, dim, generator=g, dtype=torch.float64)
    v = torch.randn(total, 1, vdim, generator=g, dtype=torch.float64)
    k[place, 0] = 3.0 * q[0, 0] / q[0, 0].norm()  # head 0 finds it; head 1 sees nothing special
    sink = torch.tensor([0.0, 0.0], dtype=torch.float64)
    want = plain_capped_attention(q, k, v, scale, cap, sink)
    got = run_attention(q, k, v, scale, cap, sink, DTYPES[dtype_name])
    tolerance = 2e-5 if dtype_name == "float32" else 3e-2
    assert torch.allclose(got, want, atol=tolerance * float(want.abs().max()))
    score = cap * math.tanh(3.0 * float(q[0, 0].norm()) / cap)  # the others' scores are near zero, the sink's is zero
    assert math.exp(score) / (math.exp(score) + total) > 0.9
    assert float((want[0, 0] - v[place, 0]).norm()) < 0.2 * float((want[0, 1] - v[place, 0]).norm())


@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("heads,kv_heads,page", [(4, 2, 8), (8, 1, 16), (12, 1, 16), (4, 4, 4)])
@pytest.mark.parametrize("news", [[1, 1, 1, 1], [90, 5, 130, 2], [1, 40, 1, 7], [400, 90, 130, 300]])
@pytest.mark.parametrize("cap", [2.0, 20.0])
def test_tensor_core_attention_with_capped_scores_and_sinks(head_dim, heads, kv_heads, page, news, cap):
    """The bfloat16 kernels on tensor cores (prompt portions by mma.sync and, for heads of 128, on tcgen05; decode by
    TMA for groups up to 8 and pages from 8 tokens, else the tiled one; mixed steps) with the cap on the scaled
    scores and learned sinks, against float64.  Queries and keys are unit vectors times sqrt(head_dim), as behind the
    unit norm; the scale makes the largest scores pass the smaller cap."""
    from test_kernels_gpu import fake_context

    from mini_engine_b200.csrc import attention_bf16, ops

    g = torch.Generator().manual_seed(head_dim + heads + page + len(news) + int(cap))
    lengths = [400, 90, 130, 300]
    scale = 8.0 / head_dim
    total_pages = sum(-(-n // page) for n in lengths) + 3
    order = torch.randperm(total_pages, generator=g).tolist()
    k_pages = torch.randn(total_pages, kv_heads, page, head_dim, generator=g).to(torch.bfloat16)
    v_pages = torch.randn(total_pages, kv_heads, page, head_dim, generator=g).to(torch.bfloat16)
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths) + 1), -1, dtype=torch.int32)
    sink = 2.0 * torch.randn(heads, generator=g)
    q_rows, want_rows, entry_of, positions = [], [], [], []
    for b, (n, new) in enumerate(zip(lengths, news)):
        q = plain.rms_norm(torch.randn(n, heads, head_dim, generator=g), None, 1e-6).to(torch.bfloat16)
        k = plain.rms_norm(torch.randn(n, kv_heads, head_dim, generator=g), None, 1e-6)
        k[n // 2] = q[n - 1, ::heads // kv_heads].float()  # one key that the last query meets at the cap
        k = k.to(torch.bfloat16)
        v = torch.randn(n, kv_heads, head_dim, generator=g).to(torch.bfloat16)
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
        for position in range(n):
            k_pages[table[b, position // page], :, position % page] = k[position]
            v_pages[table[b, position // page], :, position % page] = v[position]
        want = plain_capped_attention(q.double()[n - new :], k.double(), v.double(), scale, cap, sink.double())
        q_rows.append(q[n - new :]), want_rows.append(want)
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
        heads=heads, kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=0, sink_values=sink.cuda(), softcap=cap,
    )  # fmt: skip
    torch.cuda.synchronize()
    assert attention_bf16.take_error() == 0
    error = float((out.float().cpu() - want).abs().max()) / float(want.abs().max())
    assert error < 2e-2, f"relative error {error:.3g}"
    if cap == 2.0:  # the cap matters: without it the same kernels give another result
        ops.paged_attention(
            q=q_all, k_pages=k_pages.cuda(), v_pages=v_pages.cuda(), block_table=table.cuda(), ctx=fake_context(data), out=out,
            heads=heads, kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=0, sink_values=sink.cuda(),
        )  # fmt: skip
        assert float((out.float().cpu() - want).abs().max()) / float(want.abs().max()) > 5e-2


@pytest.mark.parametrize("heads,dim,vdim,dims", [(2, 16, 8, 16), (3, 24, 40, 8), (1, 6, 5, 2), (2, 64, 64, 64), (1, 128, 32, 32), (2, 192, 128, 64)])
def test_retention_alone_whole_and_token_by_token(heads, dim, vdim, dims):
    """The recurrence with the rotation, the key scale and a decay per head, then unit norm and gate: a whole prompt
    against the plain loop; then the same tokens in portions and one by one from the carried state (the same bits);
    a second request in the same launch starts from zero in a slot that held another state."""
    from mini_engine_b200.csrc import ops

    g = torch.Generator().manual_seed(dim + heads)
    tokens, hidden, eps = 45, 24, 1e-5
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": [0.9, 0.999, 0.5][:heads], "rot": {"base": 300.0, "dims": dims}}
    w = {"q": torch.randn(heads * dim, hidden, generator=g), "k": torch.randn(heads * dim, hidden, generator=g),
         "v": torch.randn(heads * vdim, hidden, generator=g), "g": torch.randn(heads * vdim, hidden, generator=g),
         "o": torch.eye(heads * vdim)}  # fmt: skip
    w = {key: value.double() for key, value in w.items()}
    h = torch.randn(tokens, hidden, generator=g, dtype=torch.float64)
    want, _ = plain.retention(h, w, "", m, eps)
    proj = torch.cat([h @ w[key].T for key in ("q", "k", "v", "g")], dim=1)
    columns = {"q": 0, "k": heads * dim, "v": 2 * heads * dim, "g": 2 * heads * dim + heads * vdim}
    decay = torch.tensor(m["decay"], dtype=torch.float32, device="cuda")
    state = torch.full((3, heads, dim, vdim), 7.0, dtype=torch.float32, device="cuda")  # slots hold someone's past

    chunked = ops.retention_chunked_supports(dim, vdim)
    assert chunked == (dim % 4 == 0 and vdim % 4 == 0)

    def run(first, count, slot, rows, chunk_min=0):
        positions = torch.arange(first, first + count)
        angle = positions.double().view(-1, 1) * plain.frequencies(m["rot"], h)
        table = cuda(torch.stack((torch.cos(angle), torch.sin(angle)), dim=-1), torch.float32)
        part = cuda(torch.stack((0.25 * rows, 0.75 * rows)), torch.float32)  # two partial sums
        raw = torch.empty(count, heads * vdim, dtype=torch.float32, device="cuda")
        prepared = torch.empty(count, heads * 3 * dim, dtype=torch.float32, device="cuda")
        scratch = torch.full((count // 64 + 1, heads, dim, vdim), float("nan"), dtype=torch.float32, device="cuda") if chunk_min else None
        ops.retention_scan(proj=part, columns=columns, cos_sin=table, decay=decay, k_scale=dim**-0.5, ctx=Context([count], [first], [slot]),
                           state=state, out=raw, prepared=prepared, heads=heads, dim=dim, vdim=vdim, chunk_min=chunk_min,
                           chunk_state=scratch)  # fmt: skip
        out = torch.empty(count, heads * vdim, dtype=torch.float32, device="cuda")
        ops.gla_finish(o=raw, proj=part, gate_column=columns["g"], weight=None, eps=eps, out=out, heads=heads, vdim=vdim)
        return out.cpu()

    whole = run(0, tokens, 0, proj)
    assert torch.allclose(whole.double(), want, atol=3e-5 * float(want.abs().max()))
    cuts = [0, 2, 3, 20, 21, 37, tokens]
    pieces = torch.cat([run(a, b - a, 1, proj[a:b]) for a, b in zip(cuts, cuts[1:])])
    assert torch.equal(pieces, whole)
    assert torch.equal(state[0], state[1])  # the carried state is the whole prompt's
    if chunked:  # the same in chunks of 64 tokens (a whole one and a part of one), from zero and from a carried state
        h_long = torch.randn(150, hidden, generator=g, dtype=torch.float64)
        want_long, want_state = plain.retention(h_long, w, "", m, eps)
        proj_long = torch.cat([h_long @ w[key].T for key in ("q", "k", "v", "g")], dim=1)
        for cuts in ([0, 150], [0, 70, 150], [0, 5, 69, 150], [0, 64, 128, 150]):
            got = torch.cat([run(a, b - a, 2, proj_long[a:b], chunk_min=33) for a, b in zip(cuts, cuts[1:])])
            assert torch.allclose(got.double(), want_long, atol=3e-5 * float(want_long.abs().max())), cuts
            assert torch.allclose(state[2].cpu().double(), want_state, atol=3e-5 * float(want_state.abs().max())), cuts


def test_latent_layer_and_capped_layer_against_plain(tmp_path):
    """One latent layer (neighbour pairs rotated) and one capped attention layer as whole models, far keys included."""
    for layer in (
        {"type": "latent_attention", "mixer": latent(4, 16, 16, 16, 48, 0.2, 10000.0), "mlp": None},
        # a latent of 128 and rows of 192: the sizes that the tensor-core kernels over latent rows take in bfloat16
        {"type": "latent_attention", "mixer": latent(4, 64, 64, 32, 128, 0.09, 5000.0), "mlp": None},
        # heads of 128, keys and values alike: the tensor-core attention kernels with the cap and the sink
        {"type": "attention", "mixer": attention(2, 1, 128, 128, 0.07, 6.0, rot(10000.0, 64, 2.0)), "mlp": None},
        {"type": "attention", "mixer": attention(4, 2, 32, 16, 0.3, 4.0, rot(10000.0, 16, 2.0)), "mlp": None},
    ):
        raw = {"architecture": "Bizurax", "vocab": 100, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 1.0, "layers": [layer]}
        folder = write_model(tmp_path / f"{layer['type']}_{layer['mixer']['dim']}", raw, seed=5, scale=20.0)
        requests = {"a": random_ids(1, 300, 100), "b": random_ids(2, 2, 100)}
        for dtype_name in ("float32", "bfloat16"):
            for maker in (schedules.whole, schedules.changing_portions, lambda r: schedules.tail_one_by_one(r, 32)):
                replay_and_compare(folder, dtype_name, maker(requests), requests)


# ------------------------------------------------------------- the engine's entry point, scheduler and command line


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["S", "T"])
def test_greedy_generation_through_the_engine(folders, dtype_name, name):
    """`LLMEngine.generate`: the scheduler, portions under a 48-token budget, captured decode steps.  Every generated
    token is checked teacher-forced: its plain logit lies within the tolerance of the largest one at its position."""
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
    for prompt, tokens in zip(prompts, got):
        assert len(tokens) == 24
        if dtype_name == "bfloat16":
            continue  # a routing decision that rounding turns makes another sequence: float32 carries the comparison
        logits = plain.forward(config, weights, (prompt + tokens)[:-1]).float()
        slack = 2 * TOLERANCE[dtype_name] * float(logits.abs().max())
        for i, token in enumerate(tokens):
            row = logits[len(prompt) - 1 + i]
            assert float(row.max() - row[token]) <= slack, f"token {i} of a {len(prompt)}-token prompt"
    again = engine.generate(prompts[:2], SamplingParams(max_tokens=24, ignore_eos=True))
    assert len(again) == 2 and all(len(tokens) == 24 for tokens in again)
    if dtype_name == "float32":  # slots and pages of finished requests serve new ones: the same tokens bit for bit
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
    """A pool so small that running requests are preempted: their pages and state go back, they are computed again, and
    the tokens are those of a run with room for everyone."""
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
