// Semesun as a plan of parts: a decoder whose config.json lists its layers one by one.  A layer is a mixer, either windowed
// attention (unit-norm queries and keys, a learned bias by bucketed distance, a few first tokens that stay visible, values
// blended with those of the first such layer) or a Mamba-2 state-space mixer, and an optional feed-forward, either a two-matrix
// unit with squared ReLU or routed experts (scores over all outputs, a correction that steers the choice, groups of experts,
// identity experts, clamped gated experts); pre-norm RMSNorm everywhere, no rotation, an untied head.
//
// config.json: "architecture": "Semesun", "vocab", "width", "norm": {"eps"}, "layers": [{"type", "mixer": {...}, "mlp": {...} | null}].
//   attention mixer:  heads, kv_heads, dim, vdim, scale, bias_max, mask: {size, keep_first}, v_mix, and optionally bias_rows (see below)
//   mamba2 mixer:     heads, vdim, state, groups, conv, norm_groups
//   mlp kind "dense": ff
//   mlp kind "moe":   expert: {ff, limit}, router: {experts, top, identity, scale, groups: {count, keep}}
// Tensors: embed, head, final.norm, and per layer l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*.  The number of rows of an
// attention layer's bias table is not in config.json: it is the first extent of the tensor l<i>.mix.rel, read from the
// checkpoint's header by the loader and handed to the plan as `tensor_shapes`; where there is no checkpoint yet (a folder of random
// weights is being written) the optional key `bias_rows` says it, 16 by default.
#include "velomind_b200/velomind.h"

namespace vmb {

namespace {

const json::Value& member(const json::Value& o, const char* key, const std::string& where) {
    const json::Value* v = o.find(key);
    if (!o.is_object() || !v) throw ConfigError(where + ": missing required key '" + key + "'");
    return *v;
}

const json::Value& object_member(const json::Value& o, const char* key, const std::string& where) {
    const json::Value& v = member(o, key, where);
    if (!v.is_object()) throw ConfigError(where + ": key '" + key + "' must be an object");
    return v;
}

// the first extent of a tensor, from the shapes the loader found in the checkpoint (or `fallback` where there is no checkpoint yet)
long long first_extent(const json::Value& config, const std::string& tensor, long long fallback) {
    const json::Value* shapes = config.find("tensor_shapes");
    const json::Value* s = shapes ? shapes->find(tensor) : nullptr;
    if (!s || !s->is_array() || s->as_array().empty() || !s->as_array()[0].is_integer()) return fallback;
    return s->as_array()[0].as_int();
}

ModelPlan semesun_plan(const json::Value& config, const std::string& where) {
    KeyReader top(config, where);
    const int vocab = static_cast<int>(top.integer("vocab")), width = static_cast<int>(top.integer("width"));
    const double eps = KeyReader(object_member(config, "norm", where), where + ": norm").number("eps");
    const json::Value& layers = member(config, "layers", where);
    if (!layers.is_array() || layers.as_array().empty()) throw ConfigError(where + ": key 'layers' must be a list of layers");

    auto norm = [&]() {
        json::Value a;
        a.set("size", width);
        a.set("eps", eps);
        a.set("tensor", "");                    // the prefix is the tensor's whole name
        return PartSpec{"rmsnorm", a};
    };

    ModelPlan plan;
    plan.hidden_size = width;
    plan.vocab_size = vocab;
    const int n = static_cast<int>(layers.as_array().size());
    int n_attention = 0, n_ssm = 0, n_dense = 0, n_moe = 0;
    int n_blend = 0;
    long long blend_width = -1;                  // values per token of the first blending layer (-1: none yet)
    for (int l = 0; l < n; ++l) {
        const json::Value& L = layers.as_array()[l];
        const std::string lw = format("%s: layers[%d]", where.c_str(), l);
        const json::Value& type = member(L, "type", lw);
        if (!type.is_string()) throw ConfigError(lw + ": key 'type' must be a string");
        const json::Value& mx = object_member(L, "mixer", lw);
        KeyReader m(mx, lw + ".mixer");
        BlockSpec b;
        b.prefix = format("l%d.", l);
        b.names = {{"mixer", "mix."}, {"feed_forward", "mlp."}, {"mixer_norm", "norm1"}, {"feed_forward_norm", "norm2"}};
        json::Value a;
        a.set("hidden", width);
        a.set("heads", m.integer("heads"));
        a.set("vdim", m.integer("vdim"));
        a.set("eps", eps);
        if (type.as_string() == "attention") {
            a.set("kv_heads", m.integer("kv_heads"));
            a.set("dim", m.integer("dim"));
            a.set("scale", m.number("scale"));
            const json::Value* mask = mx.find("mask");
            if (mask && !mask->is_null()) {
                if (!mask->is_object()) throw ConfigError(lw + ".mixer: key 'mask' must be an object");
                KeyReader mk(*mask, lw + ".mixer.mask");
                a.set("window", mk.integer("size"));
                a.set("keep_first", mk.integer_or("keep_first", 0, 0));
            }
            const long long far = m.integer("bias_max");
            const long long rows = first_extent(config, b.prefix + "mix.rel", m.integer_or("bias_rows", 16, 0));
            a.set("bias_rows", rows);
            a.set("bias_far", far);
            if (m.boolean_or("v_mix", false)) {
                // (key heads and value size packed into one number: both must be those of the first blending layer)
                const long long values = m.integer("kv_heads") * (1ll << 32) + m.integer("vdim");
                if (blend_width < 0) blend_width = values;
                else if (blend_width != values)
                    throw ConfigError(format("%s.mixer: v_mix blends this layer's values with the first such layer's: kv_heads and vdim must be equal (%lld x %lld here, %lld x %lld there)",
                                             lw.c_str(), values >> 32, values & 0xffffffff, blend_width >> 32, blend_width & 0xffffffff));
                a.set("v_blend", n_blend++ == 0 ? "source" : "blend");
            }
            b.mixer = PartSpec{"window_attention", a};
            ++n_attention;
        } else if (type.as_string() == "mamba2") {
            a.set("state", m.integer("state"));
            a.set("groups", m.integer_or("groups", 1));
            a.set("conv", m.integer("conv"));
            a.set("norm_groups", m.integer_or("norm_groups", 1));
            b.mixer = PartSpec{"mamba2", a};
            ++n_ssm;
        } else {
            throw ConfigError(format("%s: type '%s' is not a mixer of this architecture (attention, mamba2)", lw.c_str(), type.as_string().c_str()));
        }
        b.mixer_norm = norm();
        const json::Value* mlp = L.find("mlp");
        if (!mlp || mlp->is_null()) {
            b.arrangement = "prenorm_mixer";
            b.feed_forward = PartSpec{"none", json::Value()};
            b.feed_forward_norm = PartSpec{"none", json::Value()};
        } else {
            b.arrangement = "prenorm";
            b.feed_forward_norm = norm();
            const std::string fw = lw + ".mlp";
            const json::Value& kind = member(*mlp, "kind", fw);
            json::Value f;
            f.set("hidden", width);
            if (kind.is_string() && kind.as_string() == "dense") {
                f.set("intermediate", KeyReader(*mlp, fw).integer("ff"));
                f.set("activation", "relu_squared");
                f.set("up", "up");
                f.set("down", "down");
                b.feed_forward = PartSpec{"mlp", f};
                ++n_dense;
            } else if (kind.is_string() && kind.as_string() == "moe") {
                const json::Value& ro = object_member(*mlp, "router", fw);
                KeyReader router(ro, fw + ".router");
                KeyReader expert(object_member(*mlp, "expert", fw), fw + ".expert");
                f.set("experts", router.integer("experts"));
                f.set("top", router.integer("top"));
                f.set("ff", expert.integer("ff"));
                f.set("routing", "scored");
                f.set("identity", router.integer_or("identity", 0, 0));
                f.set("scale", router.number_or("scale", 1.0));
                const json::Value* groups = ro.find("groups");
                if (groups && !groups->is_null()) {
                    if (!groups->is_object()) throw ConfigError(fw + ".router: key 'groups' must be an object");
                    KeyReader g(*groups, fw + ".router.groups");
                    f.set("groups", g.integer("count"));
                    f.set("groups_keep", g.integer("keep"));
                }
                f.set("glu", 1);
                f.set("limit", expert.number("limit"));
                f.set("alpha", 1.702);               // the design's constant
                b.feed_forward = PartSpec{"routed_experts", f};
                ++n_moe;
            } else {
                throw ConfigError(fw + ": kind must be 'dense' or 'moe'");
            }
        }
        plan.blocks.push_back(std::move(b));
        plan.schedule.push_back(ScheduleEntry{l, -1});
    }
    json::Value e;
    e.set("vocab", vocab);
    e.set("hidden", width);
    e.set("tensor", "");
    plan.embedding = PartSpec{"token_table", e};
    plan.embedding_prefix = "embed";
    plan.final_norm = norm();
    plan.final_norm_prefix = "final.norm";
    plan.head = PartSpec{"linear", e};
    plan.head_prefix = "head";
    plan.max_positions = 0;                      // positions enter through distances only: no limit of its own
    json::Value d;
    d.set("Vocab", format("%d tokens", vocab));
    d.set("Hidden", width);
    d.set("Layers", format("%d (%d attention, %d Mamba-2)", n, n_attention, n_ssm));
    d.set("FeedForward", format("%d dense, %d routed", n_dense, n_moe));
    plan.describe = d;
    return plan;
}

struct RegisterSemesun {
    RegisterSemesun() { register_architecture("Semesun", semesun_plan); }
} register_semesun;

}  // namespace

}  // namespace vmb
