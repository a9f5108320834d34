"""Prefill and decode throughput of another design (Pimezen, Molotar, Bevadra, Bizurax) beside Qwen3 dense at equal layer sizes.

    python -m mini_engine_b200.cli.design_bench [--design pimezen|molotar|bevadra|bizurax] [--sizes 1b,8b] [--steps K] [--warmup W]
    (or: bench.py --design pimezen|molotar|bevadra|bizurax)
    python -m mini_engine_b200.cli.design_bench --design bevadra --sizes 8b --capture prompt|decode   (a few eager steps, for a profiler)

For each size both models get the same width, feed-forward width, head counts, head size, layer count
and vocabulary, seeded random bfloat16 weights, and the same two workloads: one prompt of 2,048 tokens
(device time of the step, tokens per second) and decode steps of 8 requests at 2,048-token contexts as
captured graphs.  Pimezen's softmax attention has a window of 1,024 tokens that keeps the first 64; its
linear attention has as many heads.  Beside the step times, every kernel class is timed inside one eager
prompt step and one eager decode step (CUDA events around each launch) and set against its roofline: the
longer of (algorithmic bytes / measured copy bandwidth) and (algorithmic flops / measured bfloat16 peak)
over the time it took.  One JSON line is printed.

Molotar gets four layers in the order attention, recurrence, recurrence, attention that reads the first layer's keys
and values; its attention has Qwen3's head counts and head size, a window of 1,024 tokens and half of each head
rotated; its recurrence is as wide as the model with blocks of 128 channels and four taps; its feed-forward has 8
units in 4 groups of which 2 are kept, a token uses 2 units, and a unit is half as wide as Qwen3's feed-forward, so
that a token uses as many feed-forward weights as in Qwen3 while the layer holds four times as many.

Bevadra gets four layers in the order attention, latent attention, attention that reads the first layer's keys and
values, latent attention; its attention has Qwen3's head counts and head size and a window of 1,024 tokens; its latent
attention has as many heads with 128 plain and 64 rotated query/key elements, values of 128, a key/value latent of 512
and a query latent of three eighths of the width, and the same window; its feed-forward is as wide as Qwen3's.

Bizurax gets four layers in the order attention, retention, latent attention, retention, on four residual streams; its
attention has Qwen3's head counts and head size, no window, scores capped at 30 and a learned sink; its retention has as
many heads with the key and value widths of Pimezen's linear attention; its latent attention has 128 plain and 64 rotated
query/key elements, values of 128 and a latent of 512; the attention layers have a squared-relu feed-forward one and a
half times as wide as Qwen3's (the same weights), the retention layers 8 routed units a quarter as wide of which a token
uses 2, beside a shared unit half as wide (a token uses as many feed-forward weights as in Qwen3).
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
PROMPT, CONTEXT, BATCH, BLOCK = 2048, 2048, 8, 16
WINDOW, KEEP_FIRST = 1024, 64

SIZES = {
    # width, ff, heads, kv_heads, head size, layers, vocabulary; linear attention: key and value width per head, decay rank
    "1b": dict(width=2048, ff=6144, heads=16, kv_heads=8, head_dim=128, layers=4, vocab=32768, lin_dim=64, lin_vdim=128, rank=64),
    "8b": dict(width=4096, ff=12288, heads=32, kv_heads=8, head_dim=128, layers=4, vocab=32768, lin_dim=128, lin_vdim=128, rank=64),
}
TIMED = ("biased_attention", "mixed_attention", "gla_scan", "gla_finish", "branch_sum", "paged_attention", "qk_norm_rope_store",
         "add_rmsnorm", "swiglu", "gemm_tensor_core", "gemm_tensor_core_swiglu", "embedding", "rglru", "route",
         "qk_wide_norm_rope_store", "pair_embedding", "round_rows", "gemm_tensor_core_grouped", "sort_by_unit", "gather_rows",
         "combine_rows", "add_layernorm", "latent_down_finish", "head_product", "logits_finish", "retention_scan", "hyper_step",
         "activation", "qkv_rope_unit_store")  # fmt: skip
STREAMS, ROUTED_UNITS, ROUTED_USED = 4, 8, 2
LATENT_RANK, LATENT_ROT = 512, 64
UNITS, UNITS_USED, UNIT_GROUPS, UNIT_GROUPS_KEPT = 8, 2, 4, 2
RECURRENCE_BLOCK, RECURRENCE_TAPS = 128, 4


def molotar_config(size: dict):
    from mini_engine_b200.config import MolotarConfig

    d = size["head_dim"]
    attention = {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": d, "vdim": d, "scale": d**-0.5,
                 "mask": {"size": WINDOW},
                 "rot": {"dims": d // 2, "base": 1e6, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}  # fmt: skip
    recurrence = {"width": size["width"], "blocks": size["width"] // RECURRENCE_BLOCK, "conv": RECURRENCE_TAPS}
    mlp = {"kind": "moe", "expert": {"ff": size["ff"] // UNITS_USED, "limit": 7.0},
           "router": {"experts": UNITS, "top": UNITS_USED, "scale": 1.0, "groups": {"count": UNIT_GROUPS, "keep": UNIT_GROUPS_KEPT}}}  # fmt: skip
    pattern = [("attention", attention), ("rglru", recurrence), ("rglru", recurrence), ("attention", {**attention, "kv_from": 0})]
    layers = [{"type": kind, "mixer": mixer, "mlp": mlp} for kind, mixer in (pattern * size["layers"])[: size["layers"]]]
    return MolotarConfig.from_dict({
        "architecture": "Molotar", "vocab": size["vocab"], "width": size["width"], "norm": {"eps": 1e-6}, "postln_alpha": 2.0,
        "embedding": {"scale": size["width"] ** 0.5, "bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 7}},
        "layers": layers,
    })  # fmt: skip


def bevadra_config(size: dict):
    from mini_engine_b200.config import BevadraConfig

    d, h = size["head_dim"], size["heads"]
    attention = {"heads": h, "kv_heads": size["kv_heads"], "dim": d, "vdim": d, "scale": d**-0.5, "mask": {"size": WINDOW}}
    latent = {"heads": h, "dim": d, "rot_dim": LATENT_ROT, "vdim": d, "kv_rank": LATENT_RANK, "q_rank": 3 * size["width"] // 8,
              "scale": (d + LATENT_ROT) ** -0.5, "mask": {"size": WINDOW}, "rot": {"dims": LATENT_ROT, "base": 1e4}}  # fmt: skip
    mlp = {"kind": "dense", "ff": size["ff"]}
    pattern = [("attention", attention), ("latent_attention", latent), ("attention", {**attention, "kv_from": 0}), ("latent_attention", latent)]
    layers = [{"type": kind, "mixer": mixer, "mlp": mlp} for kind, mixer in (pattern * size["layers"])[: size["layers"]]]
    return BevadraConfig.from_dict({"architecture": "Bevadra", "vocab": size["vocab"], "width": size["width"], "norm": {"eps": 1e-5},
                                    "logit_softcap": 30.0, "layers": layers})  # fmt: skip


def bizurax_config(size: dict):
    from mini_engine_b200.config import BizuraxConfig

    d, h, ff = size["head_dim"], size["heads"], size["ff"]
    attention = {"heads": h, "kv_heads": size["kv_heads"], "dim": d, "vdim": d, "scale": 8.0 / d, "softcap": 30.0,
                 "rot": {"base": 500000.0, "dims": d, "scaling": {"factor": 8.0}}}  # fmt: skip
    retention = {"heads": h, "dim": size["lin_dim"], "vdim": size["lin_vdim"], "decay": [1.0 - 2.0 ** (-5 - 6 * i / h) for i in range(h)],
                 "rot": {"base": 2e5, "dims": size["lin_dim"]}}  # fmt: skip
    latent = {"heads": h, "dim": d, "rot_dim": LATENT_ROT, "vdim": d, "kv_rank": LATENT_RANK, "scale": (d + LATENT_ROT) ** -0.5,
              "rot": {"base": 1e4, "dims": LATENT_ROT}}  # fmt: skip
    dense = {"kind": "dense", "ff": 3 * ff // 2}
    routed = {"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": ROUTED_UNITS, "top": ROUTED_USED}, "shared": {"ff": ff // 2}}
    pattern = [("attention", attention, dense), ("retention", retention, routed), ("latent_attention", latent, dense), ("retention", retention, routed)]
    layers = [{"type": kind, "mixer": mixer, "mlp": mlp} for kind, mixer, mlp in (pattern * size["layers"])[: size["layers"]]]
    return BizuraxConfig.from_dict({"architecture": "Bizurax", "vocab": size["vocab"], "width": size["width"], "norm": {"eps": 1e-6},
                                    "residual_mult": 0.5, "streams": STREAMS, "layers": layers})  # fmt: skip


def configs(size: dict, design: str = "pimezen"):
    from mini_engine_b200.config import PimezenConfig, Qwen3Config

    qwen = Qwen3Config(
        vocab_size=size["vocab"], hidden_size=size["width"], intermediate_size=size["ff"], num_hidden_layers=size["layers"],
        num_attention_heads=size["heads"], num_key_value_heads=size["kv_heads"], head_dim=size["head_dim"], rms_norm_eps=1e-6,
        rope_theta=1e6, max_position_embeddings=8192, tie_word_embeddings=True,
    )  # fmt: skip
    layer = {
        "type": "parallel",
        "mixer": {
            "left": {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": size["head_dim"], "vdim": size["head_dim"],
                     "scale": size["head_dim"] ** -0.5, "mask": {"size": WINDOW, "keep_first": KEEP_FIRST}},
            "right": {"heads": size["heads"], "dim": size["lin_dim"], "vdim": size["lin_vdim"], "tau": 8.0, "decay_rank": size["rank"]},
            "left_scale": 1.0, "right_scale": 1.0,
        },
        "mlp": {"kind": "dense", "ff": size["ff"], "limit": 7.0},
    }  # fmt: skip
    pimezen = PimezenConfig.from_dict({"architecture": "Pimezen", "vocab": size["vocab"], "width": size["width"],
                                       "norm": {"eps": 1e-6}, "layers": [layer] * size["layers"]})  # fmt: skip
    if design == "molotar":
        return {"molotar": molotar_config(size), "qwen3": qwen}
    if design == "bevadra":
        return {"bevadra": bevadra_config(size), "qwen3": qwen}
    if design == "bizurax":
        return {"bizurax": bizurax_config(size), "qwen3": qwen}
    return {"pimezen": pimezen, "qwen3": qwen}


class KernelTimes:
    """While open, every launch through the named bindings is bracketed by two CUDA events."""

    def __init__(self):
        self.events: list[tuple[str, object, object]] = []

    def __enter__(self):
        import torch

        from mini_engine_b200.csrc import ops

        self.saved = {name: getattr(ops, name) for name in TIMED}
        for name, function in self.saved.items():
            def timed(*args, _name=name, _function=function, **kwargs):
                if _name == "paged_attention" and kwargs.get("v_pages", 0) is None:
                    _name = "latent_attention"  # the same entry point over a cache of latent rows
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                result = _function(*args, **kwargs)
                end.record()
                self.events.append((_name, start, end))
                return result

            setattr(ops, name, timed)
        return self

    def __exit__(self, *exc):
        from mini_engine_b200.csrc import ops

        for name, function in self.saved.items():
            setattr(ops, name, function)

    def totals(self) -> dict[str, float]:
        import torch

        torch.cuda.synchronize()
        out: dict[str, float] = {}
        for name, start, end in self.events:
            out[name] = out.get(name, 0.0) + start.elapsed_time(end) * 1e3  # microseconds
        return out


def visible_sum(tokens_from: int, tokens_to: int, window: int | None, keep_first: int) -> int:
    """Sum over query positions [from, to) of the keys each sees."""
    total = 0
    for p in range(tokens_from, tokens_to):
        if window is None or p < window:
            total += p + 1
        else:
            total += window + min(keep_first, p - window + 1)
    return total


def rooflines(design: str, size: dict, peaks: dict) -> dict:
    """Algorithmic bytes and flops of one layer's attention-class kernels, for the prompt and for the decode step."""
    h, g, d = size["heads"], size["kv_heads"], size["head_dim"]
    bw, flops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    out = {}

    def bound(name, nbytes, nflops):
        out[name] = {"bytes": nbytes, "flops": nflops, "roofline_us": max(nbytes / bw, nflops / flops) * 1e6}

    window = WINDOW if design in ("pimezen", "molotar", "bevadra") else None
    keep = KEEP_FIRST if design == "pimezen" else 0
    seen_prompt = visible_sum(0, PROMPT, window, keep)
    seen_decode = BATCH * visible_sum(CONTEXT, CONTEXT + 1, window, keep)
    mixing = 2 * h * h if design == "pimezen" else 0  # flops per (query, key) of mixing the heads' weights
    kind = "mixed_attention" if design == "pimezen" else "paged_attention"
    bound(f"prompt.{kind}", PROMPT * (2 * h * d + 2 * g * d) * 2, seen_prompt * (4 * h * d + mixing))
    bound(f"decode.{kind}", seen_decode * g * 2 * d * 2 + BATCH * 2 * h * d * 2, seen_decode * (4 * h * d + mixing))
    if design == "pimezen":
        ld, lv, rank = size["lin_dim"], size["lin_vdim"], size["rank"]
        state = h * ld * lv * 4
        row = (2 * h * ld + h * lv + rank) * 4
        bound("prompt.gla_scan", PROMPT * (row + h * lv * 4) + 2 * state, PROMPT * h * ld * lv * 4)
        bound("decode.gla_scan", BATCH * (8 * row + h * lv * 4 + 2 * state), BATCH * h * ld * lv * 4)
    # The products of a layer (averaged over the layers): a prompt is bound by the flops of the weights a token uses,
    # a decode step by the bytes of the weights that the batch touches.
    width, ff = size["width"], size["ff"]
    if design == "molotar":
        c = width  # channels of the recurrence
        mixers = [width * (h * d + 2 * g * d + h) + h * d * width, 3 * width * c, 3 * width * c, width * (h * d + h) + h * d * width]
        mixer = sum(mixers) / len(mixers)
        unit = 3 * width * (ff // UNITS_USED)
        used = UNITS_USED * unit
        touched = UNITS * (1.0 - (1.0 - UNITS_USED / UNITS) ** BATCH) * unit
        for phase, tokens, nbytes in (("prompt", PROMPT, (mixer + UNITS * unit) * 2), ("decode", BATCH, (mixer + touched) * 2)):
            nflops = 2 * tokens * (mixer + used)
            out[f"{phase}.products"] = {"bytes": nbytes, "flops": nflops, "roofline_us": max(nbytes / bw, nflops / flops) * 1e6,
                                        "kernels": ("gemm_tensor_core", "gemm_tensor_core_grouped", "swiglu")}  # fmt: skip
        # the recurrence: the projections' sums in, the decay and the driven term out and in again, the gated state out
        gates = 2 * c * RECURRENCE_BLOCK
        bound("prompt.rglru", PROMPT * c * (2 * 4 + 4 * 4 + 2) + gates * 4, 2 * PROMPT * gates)
        bound("decode.rglru", BATCH * c * (2 * 4 + 4 * 4 + 2 + 2 * RECURRENCE_TAPS * 4) + gates * 4, 2 * BATCH * gates)
        # kernel times are averaged over all layers, of which half have an attention and half a recurrence
        for name in ("prompt.paged_attention", "decode.paged_attention", "prompt.rglru", "decode.rglru"):
            out[name] = {key: value * 0.5 for key, value in out[name].items()}
        # (the products' record counts the activation kernel of the masked form as well: Qwen3's runs in its product's epilogue)
    elif design == "bevadra":
        rank, rot, q_rank = LATENT_RANK, LATENT_ROT, 3 * width // 8
        key = rank + rot
        # attention: the gates of every element are read as well (32-bit)
        for phase, tokens in (("prompt", PROMPT), ("decode", BATCH)):
            out[f"{phase}.paged_attention"]["bytes"] += tokens * h * d * 4
        for phase, tokens, seen in (("prompt", PROMPT, seen_prompt), ("decode", BATCH, seen_decode)):
            rows = tokens if phase == "prompt" else seen  # cached rows that the step reads at least once
            bound(f"{phase}.latent_attention", (rows * key + tokens * h * (key + rank)) * 2, seen * h * 2 * (key + rank))
            # the two per-head products: queries into the latent's space, averaged latents into values
            bound(f"{phase}.head_product", (2 * h * d * rank + tokens * h * (2 * d + rot + key + rank)) * 2, 2 * tokens * 2 * h * d * rank)
        mixers = [width * (2 * h * d + 2 * g * d) + h * d * width, width * (q_rank + key + h) + q_rank * h * (d + rot) + h * d * width,
                  width * 2 * h * d + h * d * width, width * (q_rank + key + h) + q_rank * h * (d + rot) + h * d * width]  # fmt: skip
        mixer = sum(mixers) / len(mixers)
        dense = 3 * width * ff
        for phase, tokens in (("prompt", PROMPT), ("decode", BATCH)):
            nbytes, nflops = (mixer + dense) * 2, 2 * tokens * (mixer + dense)
            out[f"{phase}.products"] = {"bytes": nbytes, "flops": nflops, "roofline_us": max(nbytes / bw, nflops / flops) * 1e6,
                                        "kernels": ("gemm_tensor_core", "gemm_tensor_core_swiglu", "swiglu")}  # fmt: skip
        # kernel times are averaged over all layers, of which half have an attention and half a latent attention
        for name in [n for n in out if n.split(".")[1] in ("paged_attention", "latent_attention", "head_product")]:
            nbytes, nflops = out[name]["bytes"] * 0.5, out[name]["flops"] * 0.5
            out[name] = {"bytes": nbytes, "flops": nflops, "roofline_us": max(nbytes / bw, nflops / flops) * 1e6}
    elif design == "bizurax":
        rank, rot, key = LATENT_RANK, LATENT_ROT, LATENT_RANK + LATENT_ROT
        ld, lv = size["lin_dim"], size["lin_vdim"]
        state, row = h * ld * lv * 4, (2 * h * ld + h * lv) * 4  # a request's state; a token's q, k and v sums (32-bit)
        for phase, tokens, seen in (("prompt", PROMPT, seen_prompt), ("decode", BATCH, seen_decode)):
            rows = tokens if phase == "prompt" else seen  # cached rows that the step reads at least once
            bound(f"{phase}.latent_attention", (rows * key + tokens * h * (key + rank)) * 2, seen * h * 2 * (key + rank))
            bound(f"{phase}.head_product", (2 * h * d * rank + tokens * h * (2 * d + rot + key + rank)) * 2, 2 * tokens * 2 * h * d * rank)
            # the scan: the sums in, the rotated q, k and decays out and in again, the outputs, the state in and out
            per_request = 1 if phase == "prompt" else BATCH
            bound(f"{phase}.retention_scan", tokens * (row + 2 * 3 * h * ld * 4 + h * lv * 4) + per_request * 2 * state, tokens * h * ld * lv * 4)
            # two norms per layer: every stream in and out, the pending output in, the normed row out
            bound(f"{phase}.hyper_step", 2 * tokens * width * (2 * STREAMS * 4 + 4 + 2), 2 * tokens * width * 2 * STREAMS * STREAMS)
        mixers = [width * (h * d + 2 * g * d) + h * d * width, width * (2 * h * ld + 2 * h * lv) + h * lv * width,
                  width * (h * (d + rot) + key) + h * d * width, width * (2 * h * ld + 2 * h * lv) + h * lv * width]  # fmt: skip
        mixer = sum(mixers) / len(mixers)
        unit, shared, dense = 3 * width * (ff // 4), 3 * width * (ff // 2), 2 * width * (3 * ff // 2)
        used = 0.5 * dense + 0.5 * (ROUTED_USED * unit + shared)
        touched = 0.5 * dense + 0.5 * (ROUTED_UNITS * (1.0 - (1.0 - ROUTED_USED / ROUTED_UNITS) ** BATCH) * unit + shared)
        held = 0.5 * dense + 0.5 * (ROUTED_UNITS * unit + shared)
        for phase, tokens, nbytes in (("prompt", PROMPT, (mixer + held) * 2), ("decode", BATCH, (mixer + touched) * 2)):
            nflops = 2 * tokens * (mixer + used)
            out[f"{phase}.products"] = {"bytes": nbytes, "flops": nflops, "roofline_us": max(nbytes / bw, nflops / flops) * 1e6,
                                        "kernels": ("gemm_tensor_core", "gemm_tensor_core_grouped", "gemm_tensor_core_swiglu", "swiglu", "activation")}  # fmt: skip
        # kernel times are averaged over all layers: a quarter have an attention, a quarter a latent attention, half a retention
        share = {"paged_attention": 0.25, "latent_attention": 0.25, "head_product": 0.25, "retention_scan": 0.5}
        for name in [n for n in out if n.split(".")[1] in share]:
            factor = share[name.split(".")[1]]
            nbytes, nflops = out[name]["bytes"] * factor, out[name]["flops"] * factor
            out[name] = {"bytes": nbytes, "flops": nflops, "roofline_us": max(nbytes / bw, nflops / flops) * 1e6}
    elif design == "qwen3":
        mixer = width * (h * d + 2 * g * d) + h * d * width
        dense = 3 * width * ff
        for phase, tokens, names in (("prompt", PROMPT, ("gemm_tensor_core", "gemm_tensor_core_swiglu")),
                                     ("decode", BATCH, ("gemm_tensor_core", "gemm_tensor_core_swiglu"))):  # fmt: skip
            out[f"{phase}.products"] = {"bytes": (mixer + dense) * 2, "flops": 2 * tokens * (mixer + dense),
                                        "roofline_us": max((mixer + dense) * 2 / bw, 2 * tokens * (mixer + dense) / flops) * 1e6,
                                        "kernels": names}  # fmt: skip
    return out


def run_design(design: str, cfg, size: dict, steps: int, warmup: int, peaks: dict) -> dict:
    import torch

    from mini_engine_b200 import EngineConfig, LLMEngine
    from mini_engine_b200.csrc import ops
    from mini_engine_b200.engine.runner import StepEntry

    total_steps = steps + warmup + 8
    pages = -(-(CONTEXT + total_steps + 1) // BLOCK)
    engine = LLMEngine.from_random(cfg, seed=0, config=EngineConfig(
        block_size=BLOCK, num_blocks=BATCH * pages + 8 + PROMPT // BLOCK, max_num_seqs=BATCH, max_num_batched_tokens=PROMPT,
        max_model_len=4096, enable_prefix_caching=False, dtype=torch.bfloat16, cuda_graphs=True))  # fmt: skip
    runner, graphs, manager = engine.runner, engine.decode_graphs, engine.block_manager
    generator = torch.Generator().manual_seed(1)

    def prompt(n):
        return torch.randint(0, size["vocab"], (n,), generator=generator).tolist()

    def timed(function, repeats=3, warm=3):
        times = []
        for i in range(warm + repeats):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            function()
            end.record()
            torch.cuda.synchronize()
            if i >= warm:
                times.append(start.elapsed_time(end))
        return statistics.median(times)

    def note(text):
        print(f"[design_bench] {design} width {size['width']}: {text}", file=sys.stderr, flush=True)

    cache = manager.new_request()
    assert manager.try_allocate(cache, PROMPT)
    entry = StepEntry(cache, 0, prompt(PROMPT), (PROMPT - 1,))
    note("prompt step")
    prefill_ms = timed(lambda: runner.execute([entry]))
    note(f"prompt step {prefill_ms:.2f} ms; kernels of a prompt step")
    with KernelTimes() as kernel_times:
        runner.execute([entry])
    prompt_kernels = kernel_times.totals()
    manager.free(cache)

    note("filling the decode contexts")
    caches = []
    for _ in range(BATCH):
        c = manager.new_request()
        assert manager.try_allocate(c, CONTEXT + total_steps + 1)
        runner.execute([StepEntry(c, 0, prompt(CONTEXT), ())])
        caches.append(c)
    tokens, position = prompt(BATCH), CONTEXT

    def one_step(run):
        nonlocal position
        run([StepEntry(c, position, [tokens[i]], (0,)) for i, c in enumerate(caches)])
        position += 1

    note("decode steps")
    for _ in range(warmup):
        one_step(graphs.run)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one_step(graphs.run)
    end.record()
    torch.cuda.synchronize()
    decode_ms = start.elapsed_time(end) / steps
    note(f"decode step {decode_ms:.3f} ms; kernels of a decode step")
    one_step(runner.execute)  # an eager decode step first, so that its buffers exist
    with KernelTimes() as kernel_times:
        one_step(runner.execute)
    decode_kernels = kernel_times.totals()
    ops.raise_on_device_error()

    layers = size["layers"]
    bounds = rooflines(design, size, peaks)
    kernels = {}
    for phase, totals in (("prompt", prompt_kernels), ("decode", decode_kernels)):
        for name, microseconds in sorted(totals.items()):
            per_layer = microseconds / (layers if name not in ("embedding",) else 1)
            record = {"us_per_layer": round(per_layer, 2)}
            bound = bounds.get(f"{phase}.{name}")
            if bound:
                record["roofline_us"] = round(bound["roofline_us"], 3)
                record["of_roofline"] = round(bound["roofline_us"] / per_layer, 4)
            kernels[f"{phase}.{name}"] = record
        combined = bounds.get(f"{phase}.products")
        if combined:  # all products of a layer against one bound (gated and plain ones are separate kernel classes)
            spent = sum(totals.get(name, 0.0) for name in combined["kernels"]) / layers
            kernels[f"{phase}.products"] = {"us_per_layer": round(spent, 2), "roofline_us": round(combined["roofline_us"], 3),
                                            "of_roofline": round(combined["roofline_us"] / spent, 4) if spent else None}  # fmt: skip
    return {
        "prefill_ms": round(prefill_ms, 3), "prefill_tokens_per_s": round(PROMPT / prefill_ms * 1e3, 1),
        "decode_ms_per_step": round(decode_ms, 4), "decode_tokens_per_s": round(BATCH / decode_ms * 1e3, 1),
        "layer_weight_bytes": layer_weight_bytes(runner.model, layers), "kernels": kernels,
    }  # fmt: skip


def layer_weight_bytes(model, layers: int) -> int:
    """Bytes of one layer's weights as the device holds them (matrices bfloat16, vectors float32)."""
    import math

    total = 0
    for blk in model.blocks:
        for spec in blk.weight_specs():
            if spec.alias_of is None and not spec.optional:
                total += math.prod(spec.shape) * (2 if spec.role == "matrix" else 4)
    return total // layers


def run(sizes: list[str], steps: int, warmup: int, design: str = "pimezen") -> dict:
    import torch

    peaks_file = ROOT / "MEASURED_PEAKS.json"
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if peaks_file.is_file():
        raw = json.loads(peaks_file.read_text())
        peaks = {"hbm_gbs": float(raw.get("hbm_gbs", 6650.0)), "bf16_tflops": float(raw.get("bf16_tflops", 1590.0)), "source": "measured"}
    out = {"metric": f"prefill and decode throughput of {design.capitalize()} beside Qwen3 dense at equal layer sizes", "dtype": "bf16",
           "data": "synthetic", "workload": {"prompt_tokens": PROMPT, "decode_batch": BATCH, "decode_context": CONTEXT,
                                             "window": WINDOW, "keep_first": KEEP_FIRST, "steps": steps, "warmup": warmup},
           "peaks": peaks, "sizes": {}}  # fmt: skip
    for name in sizes:
        size = SIZES[name]
        out["sizes"][name] = {"config": size}
        for which, cfg in configs(size, design).items():
            out["sizes"][name][which] = run_design(which, cfg, size, steps, warmup, peaks)
            torch.cuda.empty_cache()
    return out


def capture_steps(design: str, size_name: str, phase: str) -> None:
    """A few eager steps of one model and nothing else, for a profiler: ``prompt`` is one 2,048-token step,
    ``decode`` fills 8 contexts of 2,048 tokens and runs three steps of one token each."""
    import torch

    from mini_engine_b200 import EngineConfig, LLMEngine
    from mini_engine_b200.csrc import ops
    from mini_engine_b200.engine.runner import StepEntry

    size = SIZES[size_name]
    cfg = configs(size, design if design != "qwen3" else "pimezen")[design]
    requests = 1 if phase == "prompt" else BATCH
    pages = -(-(CONTEXT + 16) // BLOCK)
    engine = LLMEngine.from_random(cfg, seed=0, config=EngineConfig(
        block_size=BLOCK, num_blocks=requests * pages + 8, max_num_seqs=BATCH, max_num_batched_tokens=PROMPT,
        max_model_len=4096, enable_prefix_caching=False, dtype=torch.bfloat16, cuda_graphs=False))  # fmt: skip
    runner, manager = engine.runner, engine.block_manager
    generator = torch.Generator().manual_seed(1)
    caches = []
    for _ in range(requests):
        cache = manager.new_request()
        assert manager.try_allocate(cache, CONTEXT + 16)
        runner.execute([StepEntry(cache, 0, torch.randint(0, size["vocab"], (CONTEXT,), generator=generator).tolist(), (CONTEXT - 1,))])
        caches.append(cache)
    if phase == "decode":
        for step in range(3):
            runner.execute([StepEntry(cache, CONTEXT + step, [7], (0,)) for cache in caches])
    torch.cuda.synchronize()
    ops.raise_on_device_error()


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--design", choices=["pimezen", "molotar", "bevadra", "bizurax"], default="pimezen")
    parser.add_argument("--sizes", default="1b,8b")
    parser.add_argument("--steps", type=int, default=32)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--capture", choices=["prompt", "decode"], default=None,
                        help="run only a few eager steps of --model at the first of --sizes (for a profiler) and print nothing")
    parser.add_argument("--model", default=None, help="with --capture: the design itself (default) or qwen3")
    args = parser.parse_args(argv)
    if args.capture:
        capture_steps(args.model or args.design, args.sizes.split(",")[0], args.capture)
        return 0
    print(json.dumps(run(args.sizes.split(","), args.steps, max(args.warmup, 3), args.design)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
