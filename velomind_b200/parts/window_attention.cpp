// Windowed grouped-query attention with a learned bias by distance, as a mixer.
//
//   q, k, v = W_q x, W_k x, W_v x            H query heads and G key heads of `dim`, G value heads of `vdim` (they may differ)
//   q, k <- unit-rms norm per head, times a weight vector shared by all heads
//   score(i, j) = scale q_i . k_j + rel[bucket(i - j), h]
//   i sees j  iff  j <= i and (i - j < window or j < keep_first)        window 0: every earlier key
//   softmax over the visible keys, times v, then W_o
//
// No rotation: positions enter through the bias and the mask alone.  The bias table `rel` has `bias_rows` rows (0: no bias):
// one per distance below bias_rows / 2, then rows spaced evenly in the logarithm of the distance up to `bias_far`, the last
// for everything beyond; the table from distance to row is made once on the host, in double precision.
//
// Value blending (`v_blend`): a layer with "source" leaves the values it projected under `v_blend_name` for the later layers
// of the same step; a layer with "blend" caches (1 - lambda) v + lambda v_source instead of v, lambda being its tensor `vmix`.
#include <algorithm>
#include <cmath>

#include "args.h"
#include "linear.h"

namespace vmb {

// the row of the bias table a distance reads
static int distance_row(long long n, int rows, int far) {
    const int half = rows / 2;
    if (n < half) return static_cast<int>(n);
    const double r = std::floor(std::log(static_cast<double>(n) / half) / std::log(static_cast<double>(far) / half) * (rows - half));
    return static_cast<int>(std::min<double>(rows - 1, half + r));
}

class WindowAttention : public Mixer {
public:
    WindowAttention(const json::Value& a) {
        const char* k = "window_attention";
        hidden_ = static_cast<int>(arg_int(a, "hidden", k));
        H_ = static_cast<int>(arg_int(a, "heads", k));
        G_ = static_cast<int>(arg_int(a, "kv_heads", k));
        Dk_ = static_cast<int>(arg_int(a, "dim", k));
        Dv_ = static_cast<int>(arg_int_or(a, "vdim", Dk_, k));
        scale_ = static_cast<float>(arg_number_or(a, "scale", 1.0 / std::sqrt(static_cast<double>(Dk_)), k));
        window_ = static_cast<int>(arg_int_or(a, "window", 0, k));
        keep_first_ = static_cast<int>(arg_int_or(a, "keep_first", 0, k));
        rows_ = static_cast<int>(arg_int_or(a, "bias_rows", 0, k));
        far_ = static_cast<int>(arg_int_or(a, "bias_far", 0, k));
        qk_norm_ = arg_int_or(a, "qk_norm", 1, k) != 0;
        eps_ = static_cast<float>(arg_number_or(a, "eps", 1e-6, k));
        blend_ = arg_string_or(a, "v_blend", "", k);
        blend_name_ = arg_string_or(a, "v_blend_name", "v_first", k);
        if (H_ <= 0 || G_ <= 0 || H_ % G_) throw ConfigError(format("part '%s': heads (%d) must be a multiple of kv_heads (%d)", k, H_, G_));
        if (Dk_ <= 0 || Dv_ <= 0) throw ConfigError(format("part '%s': dim and vdim must be positive", k));
        if (window_ < 0 || keep_first_ < 0) throw ConfigError(format("part '%s': window and keep_first must not be negative", k));
        if (window_ == 0) keep_first_ = 0;               // every key is visible anyway
        if (rows_ < 0 || (rows_ > 0 && (rows_ < 2 || far_ <= rows_ / 2)))
            throw ConfigError(format("part '%s': a bias table needs at least 2 rows and bias_far (%d) beyond half of them", k, far_));
        if (!blend_.empty() && blend_ != "source" && blend_ != "blend") throw ConfigError(format("part '%s': v_blend is \"source\" or \"blend\"", k));
    }

    WeightTable weight_specs() const override {
        WeightTable t;
        t["q"].shape = {static_cast<long long>(H_) * Dk_, hidden_};
        t["k"].shape = {static_cast<long long>(G_) * Dk_, hidden_};
        t["v"].shape = {static_cast<long long>(G_) * Dv_, hidden_};
        t["o"].shape = {hidden_, static_cast<long long>(H_) * Dv_};
        if (qk_norm_) {
            t["q.norm"].shape = t["k.norm"].shape = {Dk_};
            t["q.norm"].init_ones = t["k.norm"].init_ones = true;
        }
        if (rows_ > 0) t["rel"].shape = {rows_, H_};
        if (!blend_.empty()) t["vmix"].shape = {};       // (a source layer's is never read)
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        qkv_.bind({&w.at("q"), &w.at("k"), &w.at("v")}, bc);
        out_.bind({&w.at("o")}, bc);
        if (qk_norm_) {
            wq_ = bc.upload(w.at("q.norm"), DType::F32);
            wk_ = bc.upload(w.at("k.norm"), DType::F32);
        }
        if (rows_ > 0) {
            rel_ = bc.upload(w.at("rel"), DType::F32);
            table_.resize(static_cast<size_t>(far_) + 1);
            for (int n = 0; n <= far_; ++n) table_[n] = distance_row(n, rows_, far_);
            bucket_of_ = bc.upload_ints(table_);
        }
        if (blend_ == "blend") lambda_ = bc.upload(w.at("vmix"), DType::F32);
    }

    bool graph_safe() const override { return true; }

    CacheNeed cache_need() const override {
        CacheNeed n;
        n.kind = window_ > 0 ? CacheNeed::Window : CacheNeed::All;
        n.kv_heads = G_;
        n.key_dim = Dk_;
        n.value_dim = Dv_;
        n.window = window_;
        n.keep_first = keep_first_;
        return n;
    }

    long long width() const { return static_cast<long long>(H_ + G_) * Dk_ + static_cast<long long>(G_) * Dv_; }

    ops::BiasedMask mask() const {
        ops::BiasedMask m;
        if (rows_ > 0) {
            m.rel = static_cast<const float*>(rel_.ptr);
            m.bucket_of = static_cast<const int*>(bucket_of_.ptr);
            m.far = far_;
            m.rows = rows_;
        }
        m.window = window_;
        m.keep_first = keep_first_;
        return m;
    }

    // norms, blending and the cache write of a step's projected q | k | v; then attention over the cache
    void attend(StepContext& ctx, void* qkv, void* att) {
        const KVView kv = ctx.kv();
        const void* v_first = nullptr;
        void* v_keep = nullptr;
        const float* lambda = nullptr;
        if (blend_ == "source") {
            v_keep = ctx.share(blend_name_, static_cast<long long>(G_) * Dv_, ctx.act_dtype);
        } else if (blend_ == "blend") {
            const StepContext::Shared* s = ctx.shared(blend_name_);
            if (!s || s->cols != static_cast<long long>(G_) * Dv_ || s->dtype != ctx.act_dtype)
                throw Error("window_attention: no earlier layer of this step left values of this layer's size to blend in");
            v_first = s->ptr;
            lambda = static_cast<const float*>(lambda_.ptr);
        }
        ops::qkv_prepare(qkv, static_cast<int>(width()), qk_norm_ ? static_cast<const float*>(wq_.ptr) : nullptr,
                         qk_norm_ ? static_cast<const float*>(wk_.ptr) : nullptr, eps_, lambda, v_first, v_keep, ctx, kv, H_, G_, Dk_, Dv_);
        ops::attention_biased(ctx, qkv, static_cast<int>(width()), kv, att, H_, G_, Dk_, Dv_, scale_, mask());
    }

    int max_rows() const {
        return ops::skinny_max_rows(2 * std::max(qkv_.weight.rows() * qkv_.weight.cols(), out_.weight.rows() * out_.weight.cols()));
    }

    // bfloat16: the layer's norm goes into the q | k | v product (few tokens) and the residual sum into the output product
    bool can_fuse(const StepContext& ctx, const Norm& norm) const override {
        const float* nw;
        float eps;
        if (!norm.as_rms(&nw, &eps) || ctx.act_dtype != DType::BF16) return false;
        if (qkv_.weight.dtype != DType::BF16 || out_.weight.dtype != DType::BF16) return false;
        if (hidden_ % 8 || (H_ * Dv_) % 8 || width() % 8) return false;
        if (ctx.T_cap <= max_rows()) return hidden_ % 32 == 0 && (H_ * Dv_) % 32 == 0;
        return true;
    }

    void forward_fused(StepContext& ctx, float* h, Norm& norm) override {
        const float* nw = nullptr;
        float eps = 0.f;
        norm.as_rms(&nw, &eps);
        const bool skinny = ctx.T_cap <= max_rows();
        void* qkv = ctx.take_tokens(width(), DType::BF16);
        if (skinny && ctx.T_cap <= ops::SKINNY_NORM_ROWS) {
            ops::skinny_linear(h, nw, eps, qkv_.weight, ctx.T, qkv, static_cast<int>(width()), false, nullptr, ctx.err, ctx.stream);
        } else {
            void* x = ctx.take_tokens(hidden_, DType::BF16);
            norm.forward(ctx, h, nullptr, x, nullptr, 0);
            if (skinny) ops::skinny_linear(x, nullptr, 0.f, qkv_.weight, ctx.T, qkv, static_cast<int>(width()), false, nullptr, ctx.err, ctx.stream);
            else ops::linear(x, DType::BF16, hidden_, qkv_.weight, qkv, DType::BF16, ctx.T, ctx.stream);
            ctx.give(x);
        }
        void* att = ctx.take_tokens(static_cast<long long>(H_) * Dv_, DType::BF16);
        attend(ctx, qkv, att);
        ctx.give(qkv);
        if (skinny) ops::skinny_linear(att, nullptr, 0.f, out_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        else ops::linear_residual(att, static_cast<long long>(H_) * Dv_, out_.weight, h, ctx.T, ctx.stream);
        ctx.give(att);
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        void* qkv = ctx.take_tokens(width(), ctx.act_dtype);
        qkv_.apply(ctx, x, ctx.act_dtype, qkv, ctx.act_dtype, ctx.T, ctx.T_cap);
        void* att = ctx.take_tokens(static_cast<long long>(H_) * Dv_, ctx.act_dtype);
        attend(ctx, qkv, att);
        ctx.give(qkv);
        out_.apply(ctx, att, ctx.act_dtype, out, ctx.act_dtype, ctx.T, ctx.T_cap);
        ctx.give(att);
    }

private:
    int hidden_ = 0, H_ = 0, G_ = 0, Dk_ = 0, Dv_ = 0, window_ = 0, keep_first_ = 0, rows_ = 0, far_ = 0;
    float scale_ = 1.f, eps_ = 1e-6f;
    bool qk_norm_ = true;
    std::string blend_, blend_name_;
    Linear qkv_, out_;
    DeviceTensor wq_, wk_, rel_, bucket_of_, lambda_;
    std::vector<int> table_;
};

namespace {
RegisterPart reg("mixer", "window_attention", [](const json::Value& a) { return std::make_shared<WindowAttention>(a); });
}  // namespace

}  // namespace vmb
