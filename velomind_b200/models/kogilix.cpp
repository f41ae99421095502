// Kogilix as a plan of parts: a decoder whose config.json lists its layers one by one.  A layer is a mixer, either latent
// attention without positions or an mLSTM, and an optional feed-forward, either a dense gated unit (tanh-GELU) or routed
// experts (squared ReLU) with an optional gated shared expert; pre-norm RMSNorm everywhere, an untied head.
//
// config.json: "architecture": "Kogilix", "vocab", "width", "norm": {"eps"}, "layers": [{"type", "mixer": {...}, "mlp": {...} | null}].
//   latent_attention mixer: heads, dim, vdim, q_rank, kv_rank, scale, and optionally kv_from: the index of the layer whose
//                           cached latents this layer reads instead of projecting its own
//   mlstm mixer:            heads, dim, vdim, gate_cap
//   mlp kind "dense":       ff
//   mlp kind "moe":         expert: {ff}, router: {experts, top}, shared: {ff} | null
// Tensors: embed, head, final.norm, and per layer l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*.
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

ModelPlan kogilix_plan(const json::Value& config, const std::string& where) {
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
    int n_latent = 0, n_mlstm = 0, n_dense = 0, n_moe = 0;
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
        int cache_of = -1;
        json::Value a;
        a.set("hidden", width);
        a.set("heads", m.integer("heads"));
        a.set("dim", m.integer("dim"));
        a.set("vdim", m.integer("vdim"));
        a.set("eps", eps);
        if (type.as_string() == "latent_attention") {
            a.set("q_rank", m.integer("q_rank"));
            a.set("kv_rank", m.integer("kv_rank"));
            a.set("scale", m.number("scale"));
            if (m.has("kv_from")) {
                cache_of = static_cast<int>(m.integer("kv_from", 0));
                if (cache_of >= l) throw ConfigError(format("%s.mixer: kv_from %d must name an earlier layer", lw.c_str(), cache_of));
                const json::Value& src = layers.as_array()[cache_of];
                const json::Value* st = src.find("type");
                const json::Value* sm = src.find("mixer");
                if (!st || !st->is_string() || st->as_string() != "latent_attention" || !sm || (sm->find("kv_from") && !sm->find("kv_from")->is_null()))
                    throw ConfigError(format("%s.mixer: kv_from %d must name a latent-attention layer with latents of its own", lw.c_str(), cache_of));
                if (KeyReader(*sm, lw).integer("kv_rank") != m.integer("kv_rank"))
                    throw ConfigError(format("%s.mixer: kv_rank differs from that of layer %d, whose latents it reads", lw.c_str(), cache_of));
                a.set("own_latent", 0);
            }
            b.mixer = PartSpec{"latent_attention", a};
            ++n_latent;
        } else if (type.as_string() == "mlstm") {
            a.set("gate_cap", m.number("gate_cap"));
            b.mixer = PartSpec{"mlstm", a};
            ++n_mlstm;
        } else {
            throw ConfigError(format("%s: type '%s' is not a mixer of this architecture (latent_attention, mlstm)", lw.c_str(), type.as_string().c_str()));
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
                f.set("activation", "gelu_tanh");
                f.set("gate", "gate");
                f.set("up", "up");
                f.set("down", "down");
                b.feed_forward = PartSpec{"gated", f};
                ++n_dense;
            } else if (kind.is_string() && kind.as_string() == "moe") {
                KeyReader router(object_member(*mlp, "router", fw), fw + ".router");
                f.set("experts", router.integer("experts"));
                f.set("top", router.integer("top"));
                f.set("ff", KeyReader(object_member(*mlp, "expert", fw), fw + ".expert").integer("ff"));
                f.set("activation", "relu_squared");
                const json::Value* shared = mlp->find("shared");
                if (shared && !shared->is_null()) {
                    if (!shared->is_object()) throw ConfigError(fw + ": key 'shared' must be an object or null");
                    f.set("shared_ff", KeyReader(*shared, fw + ".shared").integer("ff"));
                    f.set("shared_gate", 1);
                }
                b.feed_forward = PartSpec{"routed_experts", f};
                ++n_moe;
            } else {
                throw ConfigError(fw + ": kind must be 'dense' or 'moe'");
            }
        }
        plan.blocks.push_back(std::move(b));
        plan.schedule.push_back(ScheduleEntry{l, cache_of});
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
    plan.max_positions = 0;                      // no position encoding, no limit of its own
    json::Value d;
    d.set("Vocab", format("%d tokens", vocab));
    d.set("Hidden", width);
    d.set("Layers", format("%d (%d latent attention, %d mLSTM)", n, n_latent, n_mlstm));
    d.set("FeedForward", format("%d dense, %d routed", n_dense, n_moe));
    plan.describe = d;
    return plan;
}

struct RegisterKogilix {
    RegisterKogilix() { register_architecture("Kogilix", kogilix_plan); }
} register_kogilix;

}  // namespace

}  // namespace vmb
