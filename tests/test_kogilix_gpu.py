"""The Kogilix design in the library against the plain implementation (tests/plain_kogilix.py): each mechanism alone
(through the probe architecture of the tests' plug-in, which lets one part's output reach the logits), whole models cut
into steps in several ways, crafted weights where random ones would hide a fault, and generation through the entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import kogilix_configs as C
import plain_kogilix as K
import schedules as S
import st_files

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ----------------------------------------------------------------------------- helpers
def write_model(folder, cfg, tensors, as_bf16=False):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    st_files.write(os.path.join(folder, "model.safetensors"), {k: np.asarray(v, np.float32) for k, v in tensors.items()},
                   bf16=set(tensors) if as_bf16 else ())
    return str(folder)


def rounded_to_bf16(tensors):
    """The same tensors with every value rounded to the nearest bfloat16 (still float32 arrays)."""
    return {k: (st_files.to_bf16_bits(v).astype(np.uint32) << 16).view(np.float32).reshape(np.shape(v)) for k, v in tensors.items()}


def probe_config(hidden, block, limit=4096):
    ident = {"kind": "identity", "args": {"size": hidden}}
    return {"architectures": ["ProbeForCausalLM"], "hidden": hidden, "vocab": hidden, "limit": limit,
            "embedding": {"kind": "token_table", "args": {"vocab": hidden, "hidden": hidden}}, "final_norm": ident, "head": ident,
            "blocks": [dict(block, mixer_norm=ident, feed_forward_norm=ident)]}


def mixer_block(kind, args):
    return {"arrangement": "mixer_only", "mixer": {"kind": kind, "args": args}, "feed_forward": {"kind": "none"}}


def ff_block(kind, args):
    none_mixer = {"kind": "mlstm", "args": {"hidden": args["hidden"], "heads": 1, "dim": 1, "vdim": 1, "gate_cap": 1.0, "eps": 1e-6}}
    return {"arrangement": "feed_forward_only", "mixer": none_mixer, "feed_forward": {"kind": kind, "args": args}}


def random_tensors(table, rng, std):
    out = {}
    for name, spec in table.items():
        shape = spec["shape"]
        out[name] = (1.0 + rng.uniform(-0.2, 0.2, shape)) if spec["ones"] else rng.normal(0.0, std, shape)
    return {k: v.astype(np.float32) for k, v in out.items()}


def run_cuts(engine, requests, plain, cuts, tol):
    scale = max(1.0, max(float(np.abs(v).max()) for v in plain.values()))
    for name, steps in cuts.items():
        got = S.run_steps_in_process(engine, steps)
        exp = S.expected_rows(steps, requests, plain)
        assert sorted(got) == sorted(exp), name
        worst = max(float(np.abs(got[k] - exp[k]).max()) for k in exp)
        assert worst < tol * scale, (name, worst, scale)
    assert engine.cache.slots.held_count == 0


def standard_cuts(requests):
    return {"whole": S.steps_whole(requests), "tail": S.steps_tail_one_by_one(requests, tail=9), "batches": S.steps_unequal_batches(requests),
            "sparse": S.steps_sparse_wants(requests)}


def steps_in_pieces(requests, sizes):
    """Each request alone, its prompt fed in pieces of the given sizes (cycled), every place wanted."""
    steps = []
    for rid, toks in requests.items():
        at, j = 0, 0
        while at < len(toks):
            n = min(sizes[j % len(sizes)], len(toks) - at)
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}],
                          "end": [rid] if at + n == len(toks) else []})
            at += n
            j += 1
    return steps


# ----------------------------------------------------------------------------- each mechanism alone
MECHANISMS = {
    "latent_attention": ("mixer", "latent_attention", {"hidden": 80, "heads": 3, "dim": 24, "vdim": 8, "q_rank": 40, "kv_rank": 48, "scale": 0.35, "eps": 1e-5}),
    "latent_attention_odd": ("mixer", "latent_attention", {"hidden": 56, "heads": 2, "dim": 10, "vdim": 14, "q_rank": 20, "kv_rank": 36, "scale": 0.5, "eps": 1e-6}),
    "mlstm": ("mixer", "mlstm", {"hidden": 72, "heads": 3, "dim": 12, "vdim": 20, "gate_cap": 9.0, "eps": 1e-5}),
    "mlstm_wide": ("mixer", "mlstm", {"hidden": 64, "heads": 1, "dim": 72, "vdim": 40, "gate_cap": 30.0, "eps": 1e-6}),
    # a key size that is no multiple of four and values wider than one block's 64 columns (two slices, the second one ragged)
    "mlstm_sliced": ("mixer", "mlstm", {"hidden": 64, "heads": 2, "dim": 18, "vdim": 80, "gate_cap": 12.0, "eps": 1e-5}),
    # a latent of 64 values: long prompts take the tcgen05 attention kernels, all query heads on the one latent "head"
    "latent_attention_64": ("mixer", "latent_attention", {"hidden": 64, "heads": 4, "dim": 16, "vdim": 32, "q_rank": 32, "kv_rank": 64, "scale": 0.3, "eps": 1e-6}),
    "gated_gelu": ("feed_forward", "gated", {"hidden": 64, "intermediate": 88, "activation": "gelu_tanh", "gate": "gate", "up": "up", "down": "down"}),
    "experts_shared": ("feed_forward", "routed_experts", {"hidden": 64, "experts": 6, "top": 2, "ff": 24, "shared_ff": 40}),
    "experts_top_one": ("feed_forward", "routed_experts", {"hidden": 48, "experts": 7, "top": 1, "ff": 16}),
    "experts_all": ("feed_forward", "routed_experts", {"hidden": 48, "experts": 3, "top": 3, "ff": 20, "shared_ff": 8}),
}


def plain_mechanism(name, args, x, w):
    kind = MECHANISMS[name][1]
    if kind == "latent_attention":
        return K.latent_attention(x, w, "layers.0.mixer.", args, args["eps"])
    if kind == "mlstm":
        return K.mlstm(x, w, "layers.0.mixer.", args, args["eps"])
    if kind == "gated":
        return K.gated_dense(x, w, "layers.0.feed_forward.")
    mlp = {"router": {"top": args["top"]}, "shared": {"ff": args["shared_ff"]} if args.get("shared_ff") else None}
    return K.routed_experts(x, w, "layers.0.feed_forward.", mlp)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_alone(name, dtype, toy_plugin, tmp_path):
    import velomind_b200 as vm
    role, kind, args = MECHANISMS[name]
    cfg = probe_config(args["hidden"], mixer_block(kind, args) if role == "mixer" else ff_block(kind, args))
    rng = np.random.default_rng(sum(name.encode()))
    w = random_tensors(vm.weight_table(cfg), rng, 0.25)
    if dtype == "bfloat16":
        w = rounded_to_bf16(w)              # stored as bfloat16; the plain implementation runs on the same rounded numbers
    folder = write_model(str(tmp_path / name), cfg, w, as_bf16=dtype == "bfloat16")
    engine = vm.Engine(vm.load_model(folder, dtype, "cuda:0"), 64 * 6, max_slots=3)
    requests = S.make_requests(args["hidden"], (70, 5, 130, 64, 1, 65), seed=3)
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        plain[rid] = x + plain_mechanism(name, args, x, w)
    if kind == "routed_experts":        # the test sees a wrong expert only if the routing spreads
        x = w["embed.weight"].astype(np.float64)
        assert len(set(K.route(x, w, "layers.0.feed_forward.", args["top"])[0].reshape(-1).tolist())) == args["experts"]
    cuts = standard_cuts(requests)
    cuts["pieces"] = steps_in_pieces(requests, (2, 3, 64, 1, 65))
    run_cuts(engine, requests, plain, cuts, 3e-5 if dtype == "float32" else 2e-2)


def test_a_long_prompt_over_a_latent_of_64_values(toy_plugin, tmp_path):
    """1,500 tokens: the block table is wide enough for the tcgen05 prefill attention kernels, which then serve four query
    heads on one shared latent that is key and value at once; then decode steps over the same pages."""
    import velomind_b200 as vm
    role, kind, args = MECHANISMS["latent_attention_64"]
    cfg = probe_config(64, mixer_block(kind, args))
    w = rounded_to_bf16(random_tensors(vm.weight_table(cfg), np.random.default_rng(77), 0.25))
    folder = write_model(str(tmp_path / "long"), cfg, w, as_bf16=True)
    engine = vm.Engine(vm.load_model(folder, "bfloat16", "cuda:0"), 64 * 40, max_slots=2)
    requests = S.make_requests(64, (1500, 2100), seed=6)
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        plain[rid] = x + K.latent_attention(x, w, "layers.0.mixer.", args, args["eps"])
    sparse = lambda n: sorted(set(range(0, n, 97)) | {n - 1})
    whole = [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": sparse(len(toks))}], "end": [rid]} for i, (rid, toks) in enumerate(requests.items())]
    run_cuts(engine, requests, plain, {"whole": whole, "tail": S.steps_tail_one_by_one({"r0": requests["r0"]}, tail=6)}, 2e-2)
    assert engine.counters["tc_attention_calls"] >= 3           # the prompts of all three steps took a tcgen05 kernel


def test_equal_router_logits_go_to_the_lower_index(toy_plugin, tmp_path):
    """Two experts with the same router row and bias tie at every token; the one with the lower index is chosen, in the
    few-token kernels and (bfloat16, prompts) in the grouped ones."""
    import velomind_b200 as vm
    args = {"hidden": 64, "experts": 5, "top": 2, "ff": 32}
    cfg = probe_config(64, ff_block("routed_experts", args))
    w = rounded_to_bf16(random_tensors(vm.weight_table(cfg), np.random.default_rng(41), 0.25))
    p = "layers.0.feed_forward."
    w[p + "router"][3] = w[p + "router"][1]
    w[p + "router.b"][3] = w[p + "router.b"][1]
    requests = S.make_requests(64, (90, 4), seed=5)
    chosen = K.route(w["embed.weight"].astype(np.float64), w, p, 2)[0]
    assert (chosen == 1).any() and ((chosen == 1).sum(axis=1) >= (chosen == 3).sum(axis=1)).all()     # 3 never without 1: the tie is real
    assert (chosen[:, 1] == 1).any()                  # tokens at which the tie decides the second expert
    mlp = {"router": {"top": 2}, "shared": None}
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        plain[rid] = x + K.routed_experts(x, w, p, mlp)
    for dtype, tol, as_bf16 in (("float32", 3e-5, False), ("bfloat16", 1.5e-2, True)):
        folder = write_model(str(tmp_path / dtype), cfg, w, as_bf16=as_bf16)
        engine = vm.Engine(vm.load_model(folder, dtype, "cuda:0"), 64 * 4)
        run_cuts(engine, requests, plain, {"whole": S.steps_whole(requests), "tail": S.steps_tail_one_by_one(requests, tail=3)}, tol)


def test_experts_of_many_tokens_bfloat16(toy_plugin, tmp_path):
    """Prompts group their (token, expert) pairs by expert and multiply on the tensor cores; decode steps stream each token's
    experts.  Both against the plain implementation, on bfloat16-exact inputs and weights, so that the routing is the same."""
    import velomind_b200 as vm
    args = {"hidden": 64, "experts": 6, "top": 2, "ff": 32, "shared_ff": 40}
    cfg = probe_config(64, ff_block("routed_experts", args))
    w = rounded_to_bf16(random_tensors(vm.weight_table(cfg), np.random.default_rng(31), 0.25))
    folder = write_model(str(tmp_path / "grouped"), cfg, w, as_bf16=True)
    engine = vm.Engine(vm.load_model(folder, "bfloat16", "cuda:0"), 64 * 12, max_slots=3)
    requests = S.make_requests(64, (130, 70, 300, 65), seed=4)
    mlp = {"router": {"top": 2}, "shared": {"ff": 40}}
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        plain[rid] = x + K.routed_experts(x, w, "layers.0.feed_forward.", mlp)
    cuts = {"whole": S.steps_whole(requests), "tail": S.steps_tail_one_by_one(requests, tail=20), "batches": S.steps_unequal_batches(requests)}
    run_cuts(engine, requests, plain, cuts, 1.5e-2)


def test_experts_inside_a_layer_bfloat16(toy_plugin, tmp_path):
    """A pre-norm layer whose mixer adds nothing (its output projection is zero), so that the logits are x + experts(norm(x)):
    with few tokens the router and the experts norm the residual stream themselves and add into it, with many the norm is a
    kernel of its own and the pairs are grouped; both against the plain implementation on the normed rows as bfloat16 holds them."""
    import velomind_b200 as vm
    args = {"hidden": 64, "experts": 6, "top": 2, "ff": 32, "shared_ff": 24}
    ident = {"kind": "identity", "args": {"size": 64}}
    quiet = {"kind": "mlstm", "args": {"hidden": 64, "heads": 1, "dim": 4, "vdim": 4, "gate_cap": 5.0, "eps": 1e-6}}
    cfg = {"architectures": ["ProbeForCausalLM"], "hidden": 64, "vocab": 64, "limit": 4096,
           "embedding": {"kind": "token_table", "args": {"vocab": 64, "hidden": 64}}, "final_norm": ident, "head": ident,
           "blocks": [{"arrangement": "prenorm", "mixer": quiet, "feed_forward": {"kind": "routed_experts", "args": args}, "mixer_norm": ident,
                       "feed_forward_norm": {"kind": "rmsnorm", "args": {"size": 64, "eps": 1e-5}}}]}
    w = rounded_to_bf16(random_tensors(vm.weight_table(cfg), np.random.default_rng(53), 0.25))
    w["layers.0.mixer.o"][:] = 0.0
    folder = write_model(str(tmp_path / "layer"), cfg, w, as_bf16=True)
    engine = vm.Engine(vm.load_model(folder, "bfloat16", "cuda:0"), 64 * 8, max_slots=3)
    requests = S.make_requests(64, (20, 3, 150), seed=7)
    mlp = {"router": {"top": 2}, "shared": {"ff": 24}}
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        xn = rounded_to_bf16({"x": K.rms_norm(x, w["layers.0.feed_forward_norm.weight"], 1e-5).astype(np.float32)})["x"].astype(np.float64)
        plain[rid] = x + K.routed_experts(xn, w, "layers.0.feed_forward.", mlp)
    cuts = {"whole": S.steps_whole(requests), "tail": S.steps_tail_one_by_one(requests, tail=10), "batches": S.steps_unequal_batches(requests)}
    run_cuts(engine, requests, plain, cuts, 1.5e-2)


# ----------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def kog_folders(tmp_path_factory):
    import velomind_b200 as vm
    root = tmp_path_factory.mktemp("kogilix")
    return {k: vm.write_random_model(str(root / k), C.config(k), seed=s, std=0.12, norm_jitter=0.2, dtype="float32")
            for k, s in (("a", 5), ("b", 6), ("c", 7))}


@pytest.mark.parametrize("which", ["a", "c"])
def test_whole_model_float32(which, kog_folders):
    import velomind_b200 as vm
    cfg, w = K.read_model(kog_folders[which])
    engine = vm.Engine(vm.load_model(kog_folders[which], "float32", "cuda:0"), 64 * 7, max_slots=3)     # few pages and slots: both are used again
    assert len(engine.cache.groups) == (0 if which == "c" else 2)
    requests = S.make_requests(cfg["vocab"], (50, 6, 140, 64, 2, 129), seed=8)
    plain = {rid: K.forward_logits(cfg, w, toks) for rid, toks in requests.items()}
    cuts = standard_cuts(requests)
    cuts["pieces"] = steps_in_pieces(requests, (3, 2, 64, 70))
    run_cuts(engine, requests, plain, cuts, 5e-5)
    engine.cache.check()


def test_whole_model_bfloat16(kog_folders, tmp_path):
    """The serving precision: weights rounded to bfloat16, then compared with the plain implementation on the SAME rounded
    weights.  A routed layer would choose another expert for a token whose two logits are closer than the rounding of its
    input, and the answer would then differ by more than rounding; so here every routed layer takes ALL its experts (their
    weights are still the softmax of the router's logits), and the choice itself is left to the float32 tests."""
    import velomind_b200 as vm
    cfg, w = K.read_model(kog_folders["b"])
    for layer in cfg["layers"]:
        if layer["mlp"] and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    bits = rounded_to_bf16(w)
    folder = write_model(str(tmp_path / "b16"), cfg, bits, as_bf16=True)
    engine = vm.Engine(vm.load_model(folder, "bfloat16", "cuda:0"), 64 * 16, max_slots=4)
    requests = S.make_requests(cfg["vocab"], (200, 31, 330), seed=9)
    plain = {rid: K.forward_logits(cfg, bits, toks) for rid, toks in requests.items()}
    scale = max(float(np.abs(v).max()) for v in plain.values())
    for steps in (S.steps_whole(requests), S.steps_tail_one_by_one(requests, tail=40), S.steps_unequal_batches(requests, tails=(30, 11, 45))):
        got = S.run_steps_in_process(engine, steps)
        exp = S.expected_rows(steps, requests, plain)
        err = np.concatenate([np.abs(got[k] - exp[k]).max(axis=1) for k in exp]) / scale
        # rounding alone: about one part in a hundred of the largest logit at most places, several times that at the worst of hundreds
        assert np.median(err) < 0.02 and err.max() < 0.15, (float(np.median(err)), float(err.max()))


def test_decode_steps_are_replayed_from_graphs(kog_folders):
    import velomind_b200 as vm
    cfg, w = K.read_model(kog_folders["a"])
    engine = vm.Engine(vm.load_model(kog_folders["a"], "float32", "cuda:0"), 64 * 8)
    assert engine.use_graphs
    requests = S.make_requests(cfg["vocab"], (20, 33), seed=10)
    plain = {rid: K.forward_logits(cfg, w, toks) for rid, toks in requests.items()}
    run_cuts(engine, requests, plain, {"tail": S.steps_tail_one_by_one(requests, tail=12)}, 5e-5)
    assert engine.graphs_captured > 0


# ----------------------------------------------------------------------------- crafted: one far key that decides the answer
def far_key_model(tmp_path, vm):
    """A latent-attention layer alone whose last token's query points at ONE earlier token's key in every head: without that
    key the answer is another one.  Returns (folder, args, weights, far token, asking token)."""
    args = {"hidden": 64, "heads": 2, "dim": 16, "vdim": 24, "q_rank": 32, "kv_rank": 32, "scale": 1.0, "eps": 1e-6}
    cfg = probe_config(64, mixer_block("latent_attention", args), limit=2048)
    rng = np.random.default_rng(17)
    w = random_tensors(vm.weight_table(cfg), rng, 0.3)
    p = "layers.0.mixer."
    far, ask = 11, 29
    e_far = w["embed.weight"][far].astype(np.float64)
    k_far = K.lin(K.latent_of(e_far[None], w, p, args["eps"]), w[p + "uk"])[0]
    # an input whose query (before the latent's norm rescales it) is the far token's key, head by head
    m = w[p + "uq"].astype(np.float64) @ (w[p + "dq.norm"].astype(np.float64)[:, None] * w[p + "dq"].astype(np.float64))
    w["embed.weight"][ask] = np.linalg.lstsq(m, k_far, rcond=None)[0].astype(np.float32)
    w = rounded_to_bf16(w)                             # both precisions then run the very same numbers
    # the design's score scale is a constant of the configuration: large enough that the far key outweighs 700 others together
    e = w["embed.weight"].astype(np.float64)
    q = K.lin(K.rms_norm(K.lin(e[ask][None], w[p + "dq"]), w[p + "dq.norm"], args["eps"]), w[p + "uq"]).reshape(args["heads"], args["dim"])
    k = K.lin(K.latent_of(e, w, p, args["eps"]), w[p + "uk"]).reshape(64, args["heads"], args["dim"])
    s_all = np.einsum("hd,nhd->hn", q, k)
    others = np.delete(s_all, [far, ask], axis=1)
    args["scale"] = float(np.ceil(10.0 / (s_all[:, far] - others.max(axis=1)).min()))
    assert 0 < args["scale"] < 200
    cfg = probe_config(64, mixer_block("latent_attention", args), limit=2048)
    return {"float32": write_model(str(tmp_path / "far32"), cfg, w), "bfloat16": write_model(str(tmp_path / "far16"), cfg, w, as_bf16=True)}, args, w, far, ask


@pytest.mark.parametrize("place", [0, 1, 63, 64, 65, 127, 128, 383, 384, 640])
def test_a_far_key_decides(place, toy_plugin, tmp_path):
    import velomind_b200 as vm
    folders, args, w, far, ask = far_key_model(tmp_path, vm)
    rng = np.random.default_rng(place)
    fill = [t for t in range(64) if t not in (far, ask)]
    n = 700
    toks = [int(rng.choice(fill)) for _ in range(n)]
    toks[place] = far
    toks[-1] = ask
    x = w["embed.weight"].astype(np.float64)[toks]
    y, weights = K.latent_attention(x, w, "layers.0.mixer.", args, args["eps"], return_weights=True)
    assert weights[:, -1, place].min() > 0.9          # the crafted key really carries the answer, among 700
    plain = {"r": x + y}
    requests = {"r": toks}
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 3e-2)):
        engine = vm.Engine(vm.load_model(folders[dtype], dtype, "cuda:0"), 64 * 12)
        whole = [{"step": 0, "entries": [{"id": "r", "tokens": toks, "want": [n - 1]}], "end": ["r"]}]
        decoded = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:-3], "want": []}], "end": []}] + \
                  [{"step": 1 + j, "entries": [{"id": "r", "tokens": [toks[n - 3 + j]], "want": [0] if j == 2 else []}], "end": ["r"] if j == 2 else []}
                   for j in range(3)]        # (only the asking token: at this score scale the others' answers are not stable under bfloat16)
        run_cuts(engine, requests, plain, {"whole": whole, "decoded": decoded}, tol)


# ----------------------------------------------------------------------------- crafted: a memory that does not fade
def test_matrix_memory_is_carried_far(toy_plugin, tmp_path):
    """Forget gates close to one and a soft cap that bites: what the first tokens wrote still shapes the answer hundreds of
    tokens later, through pieces, single tokens and a long run of decode steps."""
    import velomind_b200 as vm
    args = {"hidden": 48, "heads": 2, "dim": 16, "vdim": 12, "gate_cap": 4.0, "eps": 1e-6}
    cfg = probe_config(48, mixer_block("mlstm", args), limit=2048)
    rng = np.random.default_rng(23)
    w = random_tensors(vm.weight_table(cfg), rng, 0.3)
    p = "layers.0.mixer."
    w[p + "f.b"][:] = 9.0                              # capped at 4: a forget gate of sigmoid(4), a memory of about 55 tokens ...
    w[p + "f"] *= 0.05
    w[p + "i.b"][:] = (-3.0, 6.0)                      # ... one head below its floor of 0 for the maximum, one capped
    folder = write_model(str(tmp_path / "mem"), cfg, w)
    n = 420
    toks = [int(t) for t in rng.integers(0, 48, n)]
    x = w["embed.weight"].astype(np.float64)[toks]
    full = K.mlstm(x, w, p, args, args["eps"])
    cut = K.mlstm(x[60:], w, p, args, args["eps"])    # the same tokens without the first sixty
    assert np.abs(full[200:] - cut[140:]).max() > 1e-3 * np.abs(full).max()     # the test would see a lost state
    plain = {"r": x + full}
    requests = {"r": toks}
    engine = vm.Engine(vm.load_model(folder, "float32", "cuda:0"), 64 * 8, max_slots=2)
    cuts = {"whole": S.steps_whole(requests), "long decode": S.steps_tail_one_by_one(requests, tail=300),
            "pieces": steps_in_pieces(requests, (2, 5, 64, 1, 100))}
    run_cuts(engine, requests, plain, cuts, 3e-5)


# ----------------------------------------------------------------------------- through the entry points
def test_greedy_generation_through_the_entry_point(kog_folders):
    import velomind_b200 as vm
    cfg, w = K.read_model(kog_folders["a"])
    te = vm.load(kog_folders["a"], dtype="float32", max_tokens=2048)
    prompts = [[1, 2, 3, 4, 5], [100, 7], [9] * 70]
    out = te.generate(prompts, temperature=0.0, max_tokens=6, stop_tokens=())
    assert [len(r.tokens) for r in out] == [6, 6, 6]
    for prompt, r in zip(prompts, out):
        seq = list(prompt)
        for tok in r.tokens:
            row = K.forward_logits(cfg, w, seq)[-1]
            assert row[tok] >= row.max() - 1e-4, (seq, tok, int(row.argmax()))
            seq.append(tok)
    # several decode steps queued on the device give the same tokens
    again = te.generate(prompts, temperature=0.0, max_tokens=6, stop_tokens=(), steps_per_sync=4)
    assert [r.tokens for r in again] == [r.tokens for r in out]


def test_the_console_program_generates(kog_folders):
    """The library's command line takes the model folder as it takes any other: token ids in, greedy tokens out."""
    cfg, w = K.read_model(kog_folders["a"])
    want = K.generate_greedy(cfg, w, [5, 6, 7, 8], 5)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "smollm2_chat"), "--model", kog_folders["a"], "--dtype", "float32", "--temp", "0",
                           "--max-tokens", "5", "--prompt-ids", "5,6,7,8"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = [ln for ln in proc.stdout.splitlines() if ln.startswith("Output: ")][0]
    assert line == "Output: " + "".join(f"[{t}]" for t in want)


def test_trace_replay_program(kog_folders, tmp_path):
    cfg, w = K.read_model(kog_folders["a"])
    requests = S.make_requests(cfg["vocab"], (40, 3, 90), seed=12)
    plain = {rid: K.forward_logits(cfg, w, toks) for rid, toks in requests.items()}
    steps = S.steps_unequal_batches(requests, tails=(20, 2, 33))
    out = str(tmp_path / "out")
    for dtype, tol in (("float32", 5e-5), ("bfloat16", None)):
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", kog_folders["a"], "--dtype", dtype, "--out", out,
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
            else:
                assert np.isfinite(got).all()
