"""The Semesun design in the library against the plain implementation (tests/plain_semesun.py): each mechanism alone
(through the probe architecture of the tests' plug-in, which lets one part's output reach the logits), whole models cut
into steps in several ways, crafted weights where random ones would hide a fault, and generation through the entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_semesun as P
import schedules as S
import semesun_configs as C
from test_kogilix_gpu import (ff_block, mixer_block, probe_config, random_tensors, rounded_to_bf16, run_cuts, standard_cuts, steps_in_pieces,
                              write_model)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MIX, FF = "layers.0.mixer.", "layers.0.feed_forward."


def attention_args(hidden, heads, kv_heads, dim, vdim, scale, window, keep_first, rows, far, eps=1e-5):
    return {"hidden": hidden, "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "window": window,
            "keep_first": keep_first, "bias_rows": rows, "bias_far": far, "eps": eps}


def as_config(args):
    """A part's arguments in the shape the plain functions take (the configuration's own)."""
    return {"heads": args["heads"], "kv_heads": args["kv_heads"], "dim": args["dim"], "vdim": args["vdim"], "scale": args["scale"],
            "bias_max": args["bias_far"], "mask": {"size": args["window"] if args["window"] else 10 ** 9, "keep_first": args["keep_first"]}}


def moe_args(hidden, experts, identity, top, ff, limit, groups, keep, scale):
    return {"hidden": hidden, "experts": experts, "identity": identity, "top": top, "ff": ff, "routing": "scored", "groups": groups,
            "groups_keep": keep, "scale": scale, "glu": 1, "limit": limit, "alpha": 1.702}


def moe_as_config(a):
    return {"kind": "moe", "expert": {"ff": a["ff"], "limit": a["limit"]},
            "router": {"experts": a["experts"], "identity": a["identity"], "top": a["top"], "scale": a["scale"],
                       "groups": {"count": a["groups"], "keep": a["groups_keep"]}}}


def run_cuts_but_for_a_few_rows(engine, requests, plain, cuts, tol, few=0.01):
    """run_cuts for bfloat16 results of the state-space mixer.  A head whose output nearly cancels at some token (the state's answer
    against the skip term) is rounding noise that the unit norm over that head's part makes as large as a signal: the plain
    implementation in double precision does not see it, the same arithmetic with bfloat16's roundings does, to the last digit.  So
    one row in a hundred may differ, and the rest must not."""
    scale = max(1.0, max(float(np.abs(v).max()) for v in plain.values()))
    for name, steps in cuts.items():
        got = S.run_steps_in_process(engine, steps)
        exp = S.expected_rows(steps, requests, plain)
        assert sorted(got) == sorted(exp), name
        err = np.concatenate([np.abs(got[k] - exp[k]).max(axis=1) for k in exp])
        assert (err >= tol * scale).mean() <= few and np.isfinite(err).all(), (name, float((err >= tol * scale).mean()), float(err.max()), scale)
    assert engine.cache.slots.held_count == 0


# ----------------------------------------------------------------------------- each mechanism alone
MECHANISMS = {
    # keys wider than values, two query heads per key head, a window shorter than the prompts, three first tokens kept
    "attention": ("mixer", "window_attention", attention_args(80, 4, 2, 24, 8, 0.3, 50, 3, 14, 120)),
    # values wider than keys, one key head, sizes that are no multiple of 8, an odd table, more kept tokens than a page holds
    "attention_odd": ("mixer", "window_attention", attention_args(56, 3, 1, 10, 36, 0.45, 37, 70, 7, 33, 1e-6)),
    # every head its own key head, equal sizes, no kept tokens, a window of one page exactly
    "attention_page_window": ("mixer", "window_attention", attention_args(64, 2, 2, 16, 16, 0.25, 64, 0, 8, 500)),
    # no window at all (every earlier key), no bias table
    "attention_open": ("mixer", "window_attention", attention_args(64, 4, 4, 16, 32, 0.2, 0, 0, 0, 0)),
    # a window longer than every prompt, a table whose last row starts inside the window
    "attention_wide": ("mixer", "window_attention", attention_args(64, 2, 1, 32, 32, 0.2, 1000, 2, 6, 20)),
    # sizes the tensor-core kernel of prompts takes (bfloat16): keys of 64 and values of 32; keys of 96 and values of 128 with more
    # kept tokens than a page; keys of 32 and values of 16 without a table
    "attention_tiles": ("mixer", "window_attention", attention_args(128, 4, 1, 64, 32, 0.15, 50, 3, 18, 260)),
    "attention_tiles_kept_page": ("mixer", "window_attention", attention_args(96, 2, 1, 96, 128, 0.1, 100, 70, 10, 90)),
    "attention_tiles_plain": ("mixer", "window_attention", attention_args(64, 4, 4, 32, 16, 0.2, 20, 0, 0, 0)),
    # a table that reaches further than the distances the tensor-core kernel keeps in shared memory: two look-ups per score
    "attention_tiles_far_table": ("mixer", "window_attention", attention_args(64, 2, 1, 32, 32, 0.2, 90, 6, 24, 20000)),
    "mamba2": ("mixer", "mamba2", {"hidden": 72, "heads": 3, "vdim": 20, "state": 24, "groups": 1, "conv": 4, "norm_groups": 1, "eps": 1e-5}),
    # two groups, a state that is no multiple of 16, two taps, the norm in four parts
    "mamba2_groups": ("mixer", "mamba2", {"hidden": 64, "heads": 4, "vdim": 12, "state": 21, "groups": 2, "conv": 2, "norm_groups": 4, "eps": 1e-6}),
    # one wide head, a state of several slices, seven taps (longer than the shortest pieces), no convolution memory to speak of at 1
    "mamba2_wide": ("mixer", "mamba2", {"hidden": 64, "heads": 1, "vdim": 80, "state": 72, "groups": 1, "conv": 7, "norm_groups": 2, "eps": 1e-6}),
    "mamba2_one_tap": ("mixer", "mamba2", {"hidden": 48, "heads": 2, "vdim": 8, "state": 16, "groups": 2, "conv": 1, "norm_groups": 1, "eps": 1e-6}),
    "mlp_relu_squared": ("feed_forward", "mlp", {"hidden": 64, "intermediate": 88, "activation": "relu_squared", "up": "up", "down": "down"}),
    # three groups of three outputs of which two stay, two identity experts in the last group
    "experts": ("feed_forward", "routed_experts", moe_args(64, 7, 2, 3, 24, 1.2, 3, 2, 1.5)),
    "experts_top_one": ("feed_forward", "routed_experts", moe_args(48, 5, 0, 1, 16, 2.0, 1, 1, 1.0)),
    # every output is chosen: all experts and the identity expert
    "experts_all": ("feed_forward", "routed_experts", moe_args(48, 3, 1, 4, 20, 0.7, 2, 2, 2.5)),
    # groups of one: the choice among groups is the choice among experts
    "experts_single_groups": ("feed_forward", "routed_experts", moe_args(64, 4, 2, 2, 32, 1.0, 6, 3, 1.0)),
}


def plain_mechanism(name, args, x, w):
    kind = MECHANISMS[name][1]
    if kind == "window_attention":
        return P.attention(x, w, MIX, as_config(args), args["eps"])
    if kind == "mamba2":
        return P.mamba2(x, w, MIX, args, args["eps"])
    if kind == "mlp":
        return P.dense(x, w, FF)
    return P.routed_experts(x, w, FF, moe_as_config(args))


def shape_weights(kind, w, rng):
    """Random weights that let every branch show: a bias table as strong as the scores, corrections that change the choice,
    activations that reach the experts' clamps, step sizes and decays of every magnitude."""
    if kind == "window_attention" and MIX + "rel" in w:
        w[MIX + "rel"] = rng.normal(0.0, 1.0, w[MIX + "rel"].shape).astype(np.float32)
    if kind == "mamba2":
        H = w[MIX + "A_log"].shape[0]
        w[MIX + "A_log"] = np.linspace(-3.0, 1.0, H).astype(np.float32)
        w[MIX + "dt_bias"] = np.linspace(-2.0, 1.0, H).astype(np.float32)
        w[MIX + "D"] = rng.normal(0.0, 1.0, H).astype(np.float32)
        w[MIX + "conv"] = rng.normal(0.0, 0.6, w[MIX + "conv"].shape).astype(np.float32)
        # (x, B, C and dt three times as strong; not the gate z: a part of the norm whose gates are all shut is noise made large)
        inner = w[MIX + "norm"].shape[0]
        w[MIX + "in"][inner:] = (w[MIX + "in"][inner:] * 3.0).astype(np.float32)
    if kind == "routed_experts":
        n = w[FF + "correction"].shape[0]
        w[FF + "correction"] = (rng.normal(0.0, 0.6 / n, n) - 1.0).astype(np.float32)      # every choice score is negative
        w[FF + "router"] = (w[FF + "router"] * 4.0).astype(np.float32)
        for k in w:
            if k.endswith(".gate") or k.endswith(".up"):
                w[k] = (w[k] * 4.0).astype(np.float32)
    return w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_alone(name, dtype, toy_plugin, tmp_path):
    import velomind_b200 as vm
    role, kind, args = MECHANISMS[name]
    cfg = probe_config(args["hidden"], mixer_block(kind, args) if role == "mixer" else ff_block(kind, args))
    rng = np.random.default_rng(sum(name.encode()))
    w = shape_weights(kind, random_tensors(vm.weight_table(cfg), rng, 0.25), rng)
    if dtype == "bfloat16":
        w = rounded_to_bf16(w)              # stored as bfloat16; the plain implementation runs on the same rounded numbers
    folder = write_model(str(tmp_path / name), cfg, w, as_bf16=dtype == "bfloat16")
    engine = vm.Engine(vm.load_model(folder, dtype, "cuda:0"), 64 * 6, max_slots=3)
    requests = S.make_requests(args["hidden"], (70, 5, 130, 64, 1, 65), seed=3)
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        plain[rid] = x + plain_mechanism(name, args, x, w)
    if kind == "routed_experts":        # the test sees a wrong expert only if the routing spreads, identity experts included
        x = w["embed.weight"].astype(np.float64)
        chosen = P.route(x, w, FF, moe_as_config(args)["router"])[0]
        assert len(set(chosen.reshape(-1).tolist())) == args["experts"] + args["identity"]
    cuts = standard_cuts(requests)
    cuts["pieces"] = steps_in_pieces(requests, (2, 3, 64, 1, 65))
    # (bfloat16: a token whose two best choice scores are closer than its input's rounding may take another expert; the inputs here
    #  are bfloat16-exact, so both sides route the same numbers)
    #  float32: the recurrence's sums over the state cancel (terms of both signs, many times the size of their sum), which costs it
    #  a digit that the other mechanisms keep)
    if kind == "mamba2" and dtype == "bfloat16":
        run_cuts_but_for_a_few_rows(engine, requests, plain, cuts, 2.5e-2)
    else:
        run_cuts(engine, requests, plain, cuts, (1e-4 if kind == "mamba2" else 3e-5) if dtype == "float32" else 2.5e-2)
    engine.cache.check()


def test_an_excluded_group_counts_as_minus_infinity():
    """Choice scores below zero: a group that is left out must not come back as a score of zero."""
    rng = np.random.default_rng(5)
    a = moe_args(32, 6, 0, 2, 8, 1.0, 3, 1, 1.0)
    w = {FF + "router": rng.normal(0, 1, (6, 32)), FF + "correction": np.full(6, -3.0)}
    x = rng.normal(0, 1, (200, 32))
    chosen, weights = P.route(x, w, FF, moe_as_config(a)["router"])
    assert ((chosen[:, 0] // 2) == (chosen[:, 1] // 2)).all()      # both from the one group that stays
    assert len(set((chosen[:, 0] // 2).tolist())) == 3 and (weights > 0).all()


def test_routing_on_the_gpu_with_negative_scores_and_ties(toy_plugin, tmp_path):
    """The same on the GPU, with two outputs whose router rows and corrections are equal (the lower index wins) and one group
    of three that stays; few tokens and (bfloat16) the grouped kernels of prompts."""
    import velomind_b200 as vm
    args = moe_args(64, 7, 2, 2, 32, 1.5, 3, 1, 2.0)
    cfg = probe_config(64, ff_block("routed_experts", args))
    rng = np.random.default_rng(41)
    w = random_tensors(vm.weight_table(cfg), rng, 0.25)
    w[FF + "router"] = (w[FF + "router"] * 4.0).astype(np.float32)
    w[FF + "correction"][:] = -2.0
    w[FF + "router"][4] = w[FF + "router"][3]          # a tie inside the middle group
    w[FF + "router"][8] = w[FF + "router"][7]          # and between an expert's neighbour and an identity expert
    w = rounded_to_bf16(w)
    requests = S.make_requests(64, (150, 4), seed=5)
    chosen = P.route(w["embed.weight"].astype(np.float64), w, FF, moe_as_config(args)["router"])[0]
    assert ((chosen // 3).min(axis=1) == (chosen // 3).max(axis=1)).all() and len(set((chosen // 3).reshape(-1).tolist())) == 3
    assert (chosen == 3).any() and ((chosen == 3).sum(axis=1) >= (chosen == 4).sum(axis=1)).all()
    assert (chosen >= 7).any()
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        plain[rid] = x + P.routed_experts(x, w, FF, moe_as_config(args))
    for dtype, tol, as_bf16 in (("float32", 3e-5, False), ("bfloat16", 2e-2, True)):
        folder = write_model(str(tmp_path / dtype), cfg, w, as_bf16=as_bf16)
        engine = vm.Engine(vm.load_model(folder, dtype, "cuda:0"), 64 * 4)
        run_cuts(engine, requests, plain, {"whole": S.steps_whole(requests), "tail": S.steps_tail_one_by_one(requests, tail=3)}, tol)


def test_experts_of_many_tokens_bfloat16(toy_plugin, tmp_path):
    """Prompts group their (token, expert) pairs by expert and multiply on the tensor cores (mma.sync tiles below 256 tokens of
    capacity, tcgen05 tiles from there); identity experts join in the combining kernel; decode steps stream each token's experts."""
    import velomind_b200 as vm
    args = moe_args(64, 6, 2, 3, 64, 1.2, 4, 3, 1.5)
    cfg = probe_config(64, ff_block("routed_experts", args))
    rng = np.random.default_rng(31)
    w = rounded_to_bf16(shape_weights("routed_experts", random_tensors(vm.weight_table(cfg), rng, 0.25), rng))
    folder = write_model(str(tmp_path / "grouped"), cfg, w, as_bf16=True)
    engine = vm.Engine(vm.load_model(folder, "bfloat16", "cuda:0"), 64 * 12, max_slots=3)
    requests = S.make_requests(64, (130, 70, 300, 65), seed=4)
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        plain[rid] = x + P.routed_experts(x, w, FF, moe_as_config(args))
    cuts = {"whole": S.steps_whole(requests), "tail": S.steps_tail_one_by_one(requests, tail=20), "batches": S.steps_unequal_batches(requests)}
    run_cuts(engine, requests, plain, cuts, 2.5e-2)


# ----------------------------------------------------------------------------- crafted: one key that decides the answer
def deciding_key_model(tmp_path, vm, window, keep_first, dim=16, vdim=24):
    """An attention layer alone whose asking token's query points at ONE other token's key in every head: where the mask lets
    that key through it carries the answer, where not the answer is another one.  Returns (folders, args, weights, key token, asking token)."""
    args = attention_args(64, 2, 1, dim, vdim, 1.0, window, keep_first, 10, 300, 1e-6)
    cfg = probe_config(64, mixer_block("window_attention", args), limit=4096)
    rng = np.random.default_rng(17)
    w = random_tensors(vm.weight_table(cfg), rng, 0.3)
    w[MIX + "q.norm"][:] = 1.0
    w[MIX + "k.norm"][:] = 1.0
    w[MIX + "rel"] = rng.normal(0.0, 0.5, w[MIX + "rel"].shape).astype(np.float32)
    key, ask = 11, 29
    k_key = P.lin(w["embed.weight"][key].astype(np.float64)[None], w[MIX + "k"])[0]          # the one key head, before its norm
    # an input whose queries (before the norm rescales them) are that key, in both heads
    w["embed.weight"][ask] = np.linalg.lstsq(w[MIX + "q"].astype(np.float64), np.concatenate([k_key, k_key]), rcond=None)[0].astype(np.float32)
    w = rounded_to_bf16(w)
    # unit-norm queries and keys: the aligned score is dim * scale, the others are spread around zero; dim * scale = 48 lets the key
    # outweigh hundreds of others together
    args["scale"] = 48.0 / dim
    cfg = probe_config(64, mixer_block("window_attention", args), limit=4096)
    folders = {"float32": write_model(str(tmp_path / "key32"), cfg, w), "bfloat16": write_model(str(tmp_path / "key16"), cfg, w, as_bf16=True)}
    return folders, args, w, key, ask


# window 100, five first tokens kept, 400 tokens, the asking token last (place 399): the window's edge lies between 299 and 300
@pytest.mark.parametrize("place,seen", [(0, True), (4, True), (5, False), (63, False), (64, False), (150, False), (299, False), (300, True),
                                        (301, True), (319, True), (320, True), (383, True), (384, True), (398, True)])
@pytest.mark.parametrize("dims", [(16, 24), (32, 16)])      # the plain kernel; the tensor-core kernel of bfloat16 prompts
def test_a_key_decides_where_the_mask_lets_it(place, seen, dims, toy_plugin, tmp_path):
    import velomind_b200 as vm
    folders, args, w, key, ask = deciding_key_model(tmp_path, vm, 100, 5, *dims)
    rng = np.random.default_rng(place)
    fill = [t for t in range(64) if t not in (key, ask)]
    n = 400
    toks = [int(rng.choice(fill)) for _ in range(n)]
    toks[place] = key
    toks[-1] = ask
    x = w["embed.weight"].astype(np.float64)[toks]
    y, weights = P.attention(x, w, MIX, as_config(args), args["eps"], return_weights=True)
    if seen:
        assert weights[:, -1, place].min() > 0.9          # the crafted key really carries the answer
    else:
        assert weights[:, -1, place].max() == 0.0
    plain = {"r": x + y}
    requests = {"r": toks}
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 3e-2)):
        engine = vm.Engine(vm.load_model(folders[dtype], dtype, "cuda:0"), 64 * 8)
        whole = [{"step": 0, "entries": [{"id": "r", "tokens": toks, "want": [n - 1]}], "end": ["r"]}]
        decoded = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:-3], "want": []}], "end": []}] + \
                  [{"step": 1 + j, "entries": [{"id": "r", "tokens": [toks[n - 3 + j]], "want": [0] if j == 2 else []}], "end": ["r"] if j == 2 else []}
                   for j in range(3)]
        pieces = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:250], "want": []}], "end": []},
                  {"step": 1, "entries": [{"id": "r", "tokens": toks[250:398], "want": []}], "end": []},
                  {"step": 2, "entries": [{"id": "r", "tokens": toks[398:], "want": [1]}], "end": ["r"]}]
        run_cuts(engine, requests, plain, {"whole": whole, "decoded": decoded, "pieces": pieces}, tol)
        engine.cache.check()


def test_the_window_passes_over_decoded_tokens(toy_plugin, tmp_path):
    """The deciding key sits early in the decoded tail: the asking token comes again and again, first inside the key's reach, then
    outside it, while pages fall out of the window and come back to the pool."""
    import velomind_b200 as vm
    folders, args, w, key, ask = deciding_key_model(tmp_path, vm, 70, 2)
    rng = np.random.default_rng(3)
    fill = [t for t in range(64) if t not in (key, ask)]
    toks = [int(rng.choice(fill)) for _ in range(330)]
    toks[1] = key                                          # a kept first token: always seen
    toks[200] = key
    for at in (230, 269, 270, 271, 329):                   # 269 is the last place that sees 200
        toks[at] = ask
    x = w["embed.weight"].astype(np.float64)[toks]
    y, weights = P.attention(x, w, MIX, as_config(args), args["eps"], return_weights=True)
    assert weights[:, 269, 200].min() > 0.3 and weights[:, 270, 200].max() == 0.0 and weights[:, 329, 1].min() > 0.9
    plain = {"r": x + y}
    requests = {"r": toks}
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 3e-2)):
        engine = vm.Engine(vm.load_model(folders[dtype], dtype, "cuda:0"), 64 * 4)        # four pages: the prompt alone would need six
        steps = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:64], "want": []}], "end": []},
                 {"step": 1, "entries": [{"id": "r", "tokens": toks[64:190], "want": []}], "end": []}]
        for at in range(190, 330):
            steps.append({"step": len(steps), "entries": [{"id": "r", "tokens": [toks[at]], "want": [0] if toks[at] == ask else []}],
                          "end": ["r"] if at == 329 else []})
        run_cuts(engine, requests, plain, {"decoded": steps}, tol)
        engine.cache.check()


# ----------------------------------------------------------------------------- crafted: a state that does not fade
def test_the_state_is_carried_far(toy_plugin, tmp_path):
    """Decays close to one: what the first tokens wrote still shapes the answer hundreds of tokens later, through pieces smaller
    than the convolution, single tokens and a long run of decode steps."""
    import velomind_b200 as vm
    args = {"hidden": 48, "heads": 2, "vdim": 12, "state": 20, "groups": 1, "conv": 4, "norm_groups": 1, "eps": 1e-6}
    cfg = probe_config(48, mixer_block("mamba2", args), limit=2048)
    rng = np.random.default_rng(23)
    w = random_tensors(vm.weight_table(cfg), rng, 0.3)
    w[MIX + "A_log"][:] = (-5.0, -3.5)                     # a memory of hundreds of tokens
    w[MIX + "dt_bias"][:] = (-1.0, 0.5)
    w[MIX + "D"][:] = 0.1
    folder = write_model(str(tmp_path / "mem"), cfg, w)
    n = 420
    toks = [int(t) for t in rng.integers(0, 48, n)]
    x = w["embed.weight"].astype(np.float64)[toks]
    full = P.mamba2(x, w, MIX, args, args["eps"])
    cut = P.mamba2(x[60:], w, MIX, args, args["eps"])      # the same tokens without the first sixty
    assert np.abs(full[300:] - cut[240:]).max() > 1e-3 * np.abs(full).max()     # the test would see a lost state
    plain = {"r": x + full}
    requests = {"r": toks}
    engine = vm.Engine(vm.load_model(folder, "float32", "cuda:0"), 64 * 8, max_slots=2)
    cuts = {"whole": S.steps_whole(requests), "long decode": S.steps_tail_one_by_one(requests, tail=300),
            "pieces": steps_in_pieces(requests, (2, 5, 64, 1, 100, 3))}
    run_cuts(engine, requests, plain, cuts, 3e-5)


def test_a_slot_that_is_used_again_starts_from_nothing(toy_plugin, tmp_path):
    """One slot: every request inherits the slot of the one before, whose state and convolution inputs must be gone."""
    import velomind_b200 as vm
    name = "mamba2_groups"
    role, kind, args = MECHANISMS[name]
    cfg = probe_config(args["hidden"], mixer_block(kind, args))
    rng = np.random.default_rng(9)
    w = shape_weights(kind, random_tensors(vm.weight_table(cfg), rng, 0.25), rng)
    folder = write_model(str(tmp_path / name), cfg, w)
    engine = vm.Engine(vm.load_model(folder, "float32", "cuda:0"), 64 * 3, max_slots=1)
    requests = S.make_requests(args["hidden"], (40, 3, 90, 1, 2), seed=13)
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        plain[rid] = x + P.mamba2(x, w, MIX, args, args["eps"])
    run_cuts(engine, requests, plain, {"whole": S.steps_whole(requests), "tail": S.steps_tail_one_by_one(requests, tail=2)}, 3e-5)


# ----------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def sem_folders(tmp_path_factory):
    import velomind_b200 as vm
    root = tmp_path_factory.mktemp("semesun")
    out = {}
    for k, s in (("a", 5), ("b", 6), ("c", 7)):
        folder = vm.write_random_model(str(root / k), C.config(k), seed=s, std=0.12, norm_jitter=0.2, dtype="float32")
        cfg, w = P.read_model(folder)
        rng = np.random.default_rng(s)
        for name in w:                      # blending that shows, bias tables as strong as the scores, corrections that matter
            if name.endswith(".vmix"):
                w[name] = np.asarray(0.35 + 0.1 * rng.random(), np.float32)
            if name.endswith(".rel"):
                w[name] = rng.normal(0.0, 0.8, w[name].shape).astype(np.float32)
            if name.endswith(".correction"):
                w[name] = rng.normal(0.0, 0.3 / w[name].shape[0], w[name].shape).astype(np.float32)
            if name.endswith(".A_log"):
                w[name] = np.linspace(-3.0, 0.5, w[name].shape[0]).astype(np.float32)
        out[k] = write_model(folder, cfg, w)
    return out


@pytest.mark.parametrize("which", ["a", "c"])
def test_whole_model_float32(which, sem_folders):
    import velomind_b200 as vm
    cfg, w = P.read_model(sem_folders[which])
    engine = vm.Engine(vm.load_model(sem_folders[which], "float32", "cuda:0"), 64 * 7, max_slots=3)     # few pages and slots: both are used again
    assert len(engine.cache.groups) == (0 if which == "c" else 3)
    requests = S.make_requests(cfg["vocab"], (50, 6, 140, 64, 2, 129), seed=8)
    plain = {rid: P.forward_logits(cfg, w, toks) for rid, toks in requests.items()}
    cuts = standard_cuts(requests)
    cuts["pieces"] = steps_in_pieces(requests, (3, 2, 64, 70))
    run_cuts(engine, requests, plain, cuts, 5e-5)
    engine.cache.check()


def test_blending_reaches_the_answer(sem_folders):
    """The whole-model tests would pass with the blending left out only if it did not matter: it does."""
    cfg, w = P.read_model(sem_folders["a"])
    toks = S.make_requests(cfg["vocab"], (40,), seed=2)["r0"]
    with_blend = P.forward_logits(cfg, w, toks)
    w2 = dict(w)
    w2["l3.mix.vmix"] = np.asarray(0.0, np.float32)
    assert np.abs(P.forward_logits(cfg, w2, toks) - with_blend).max() > 1e-2 * np.abs(with_blend).max()


@pytest.mark.parametrize("which", ["a", "b"])      # sizes that only the plain kernels take; sizes the tensor-core kernels take
def test_whole_model_bfloat16(which, sem_folders, tmp_path):
    """The serving precision: weights rounded to bfloat16, then compared with the plain implementation on the SAME rounded
    weights.  A routed layer would choose another expert for a token whose two choice scores are closer than the rounding of
    its input, and the answer would then differ by more than rounding; so here every routed layer takes ALL its outputs (their
    weights are still the scores), and the choice itself is left to the float32 tests."""
    import velomind_b200 as vm
    cfg, w = P.read_model(sem_folders[which])
    for layer in cfg["layers"]:
        if layer["mlp"] and layer["mlp"]["kind"] == "moe":
            r = layer["mlp"]["router"]
            r["top"] = r["experts"] + r["identity"]
            r["groups"]["keep"] = r["groups"]["count"]
    bits = rounded_to_bf16(w)
    folder = write_model(str(tmp_path / "b16"), cfg, bits, as_bf16=True)
    engine = vm.Engine(vm.load_model(folder, "bfloat16", "cuda:0"), 64 * 16, max_slots=4)
    requests = S.make_requests(cfg["vocab"], (200, 31, 330), seed=9)
    plain = {rid: P.forward_logits(cfg, bits, toks) for rid, toks in requests.items()}
    scale = max(float(np.abs(v).max()) for v in plain.values())
    for steps in (S.steps_whole(requests), S.steps_tail_one_by_one(requests, tail=40), S.steps_unequal_batches(requests, tails=(30, 11, 45))):
        got = S.run_steps_in_process(engine, steps)
        exp = S.expected_rows(steps, requests, plain)
        err = np.concatenate([np.abs(got[k] - exp[k]).max(axis=1) for k in exp]) / scale
        assert np.median(err) < 0.02 and err.max() < 0.15, (float(np.median(err)), float(err.max()))
    engine.cache.check()


def test_decode_steps_are_replayed_from_graphs(sem_folders):
    import velomind_b200 as vm
    cfg, w = P.read_model(sem_folders["a"])
    engine = vm.Engine(vm.load_model(sem_folders["a"], "float32", "cuda:0"), 64 * 8)
    assert engine.use_graphs
    requests = S.make_requests(cfg["vocab"], (20, 33), seed=10)
    plain = {rid: P.forward_logits(cfg, w, toks) for rid, toks in requests.items()}
    run_cuts(engine, requests, plain, {"tail": S.steps_tail_one_by_one(requests, tail=12)}, 5e-5)
    assert engine.graphs_captured > 0


# ----------------------------------------------------------------------------- through the entry points
def test_greedy_generation_through_the_entry_point(sem_folders):
    import velomind_b200 as vm
    cfg, w = P.read_model(sem_folders["a"])
    te = vm.load(sem_folders["a"], dtype="float32", max_tokens=2048)
    prompts = [[1, 2, 3, 4, 5], [100, 7], [9] * 70]
    out = te.generate(prompts, temperature=0.0, max_tokens=6, stop_tokens=())
    assert [len(r.tokens) for r in out] == [6, 6, 6]
    for prompt, r in zip(prompts, out):
        seq = list(prompt)
        for tok in r.tokens:
            row = P.forward_logits(cfg, w, seq)[-1]
            assert row[tok] >= row.max() - 1e-4, (seq, tok, int(row.argmax()))
            seq.append(tok)
    # several decode steps queued on the device give the same tokens
    again = te.generate(prompts, temperature=0.0, max_tokens=6, stop_tokens=(), steps_per_sync=4)
    assert [r.tokens for r in again] == [r.tokens for r in out]


def test_the_console_program_generates(sem_folders):
    cfg, w = P.read_model(sem_folders["a"])
    want = P.generate_greedy(cfg, w, [5, 6, 7, 8], 5)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "smollm2_chat"), "--model", sem_folders["a"], "--dtype", "float32", "--temp", "0",
                           "--max-tokens", "5", "--prompt-ids", "5,6,7,8"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = [ln for ln in proc.stdout.splitlines() if ln.startswith("Output: ")][0]
    assert line == "Output: " + "".join(f"[{t}]" for t in want)


def test_trace_replay_program(sem_folders, tmp_path):
    cfg, w = P.read_model(sem_folders["a"])
    requests = S.make_requests(cfg["vocab"], (40, 3, 90), seed=12)
    plain = {rid: P.forward_logits(cfg, w, toks) for rid, toks in requests.items()}
    steps = S.steps_unequal_batches(requests, tails=(20, 2, 33))
    out = str(tmp_path / "out")
    for dtype, tol in (("float32", 5e-5), ("bfloat16", None)):
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", sem_folders["a"], "--dtype", dtype, "--out", out,
                               "--max-tokens", str(64 * 6)], input=S.to_jsonl(steps), text=True, capture_output=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]
        want = S.expected_rows(steps, requests, plain)
        scale = max(1.0, max(float(np.abs(v).max()) for v in want.values()))
        for step, rows in want.items():
            got = np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
            assert got.shape == rows.shape
            if tol is not None:
                assert float(np.abs(got - rows).max()) <= tol * scale, step
