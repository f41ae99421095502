// Latent attention without positions, as a mixer: queries and keys/values both pass through a low-rank latent, and the
// key/value latent is all the cache keeps of a token.
//
//   c_q = rmsnorm(W_dq x) ;  q_h = W_uq,h c_q                       (heads h, `dim` values each)
//   c   = rmsnorm(W_dkv x)                                           (kv_rank values: the cached row)
//   k_h = W_uk,h c ;  v_h = W_uv,h c ;  score = scale (q_h . k_h) ;  causal softmax ;  out = W_o concat_h(sum_j p_j v_h,j)
//
// Since q_h . (W_uk,h c_j) = (W_uk,h^T q_h) . c_j and sum_j p_j W_uv,h c_j = W_uv,h (sum_j p_j c_j), the up-projections move to
// the query's and the output's side: attention runs with one shared "key/value head", the latent itself, as key AND value,
// and keys and values are never made.  That is the multi-query form the attention kernels of this library already serve
// (query heads that share a kv head), so prompts and decode steps use the same kernels as grouped-query attention.
//
// A layer may read another run's latents (the schedule's `cache_of`): it then has no W_dkv of its own, and writes nothing.
#include <algorithm>
#include <cmath>

#include "args.h"
#include "linear.h"

namespace vmb {

class LatentAttention : public Mixer {
public:
    LatentAttention(int hidden, int heads, int dim, int vdim, int q_rank, int kv_rank, double scale, double eps, bool own_latent)
        : hidden_(hidden), H_(heads), D_(dim), V_(vdim), Rq_(q_rank), Rkv_(kv_rank), own_(own_latent),
          scale_(scale > 0 ? static_cast<float>(scale) : static_cast<float>(1.0 / std::sqrt(static_cast<double>(dim)))), eps_(static_cast<float>(eps)) {}

    WeightTable weight_specs() const override {
        WeightTable t;
        t["dq"].shape = {Rq_, hidden_};
        t["dq.norm"].shape = {Rq_};
        t["dq.norm"].init_ones = true;
        t["uq"].shape = {static_cast<long long>(H_) * D_, Rq_};
        if (own_) {
            t["dkv"].shape = {Rkv_, hidden_};
            t["dkv.norm"].shape = {Rkv_};
            t["dkv.norm"].init_ones = true;
        }
        t["uk"].shape = {static_cast<long long>(H_) * D_, Rkv_};
        t["uv"].shape = {static_cast<long long>(H_) * V_, Rkv_};
        t["o"].shape = {hidden_, static_cast<long long>(H_) * V_};
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        if (own_) down_.bind({&w.at("dq"), &w.at("dkv")}, bc);
        else down_.bind({&w.at("dq")}, bc);
        q_norm_ = bc.upload(w.at("dq.norm"), DType::F32);
        if (own_) kv_norm_ = bc.upload(w.at("dkv.norm"), DType::F32);
        up_q_.bind({&w.at("uq")}, bc);
        up_k_ = bc.upload(w.at("uk"), bc.dtype);          // the per-head products want one dtype for both operands
        up_v_ = bc.upload(w.at("uv"), bc.dtype);
        out_.bind({&w.at("o")}, bc);
    }

    bool graph_safe() const override { return true; }

    CacheNeed cache_need() const override {
        CacheNeed n;
        n.kind = CacheNeed::All;
        n.kv_heads = 1;
        n.key_dim = Rkv_;
        n.value_dim = 0;                                   // the latent is key and value at once
        return n;
    }

    // Few tokens (decode steps) in bfloat16: the weight-streaming products of this library, with the layer's norm taken into
    // the down-projection and the residual sum into the output projection.
    int max_rows() const {
        long long most = std::max(down_.weight.rows() * down_.weight.cols(), out_.weight.rows() * out_.weight.cols());
        most = std::max(most, up_q_.weight.rows() * up_q_.weight.cols());
        return std::min(ops::skinny_max_rows(2 * most), ops::SKINNY_NORM_ROWS);
    }

    bool can_fuse(const StepContext& ctx, const Norm& norm) const override {
        const float* nw;
        float eps;
        if (!norm.as_rms(&nw, &eps) || ctx.act_dtype != DType::BF16 || ctx.T_cap > max_rows()) return false;
        if (down_.weight.dtype != DType::BF16 || up_q_.weight.dtype != DType::BF16 || out_.weight.dtype != DType::BF16) return false;
        return hidden_ % 32 == 0 && Rq_ % 32 == 0 && (H_ * V_) % 32 == 0 && (Rq_ + (own_ ? Rkv_ : 0)) % 8 == 0 && (H_ * D_) % 8 == 0 && hidden_ % 8 == 0;
    }

    void forward_fused(StepContext& ctx, float* h, Norm& norm) override {
        const float* nw = nullptr;
        float eps = 0.f;
        norm.as_rms(&nw, &eps);
        KVView kv = ctx.kv();
        if (kv.owns != own_) throw ConfigError("a latent-attention layer and its schedule disagree about whose latents it reads");
        const int down_cols = Rq_ + (own_ ? Rkv_ : 0);
        float* down = static_cast<float*>(ctx.take_tokens(down_cols, DType::F32));
        ops::skinny_linear(h, nw, eps, down_.weight, ctx.T, down, down_cols, true, nullptr, ctx.err, ctx.stream);
        void* cq = ctx.take_tokens(Rq_, DType::BF16);
        ops::latent_norm_write(down, down_cols, Rq_, Rkv_, static_cast<const float*>(q_norm_.ptr), own_ ? static_cast<const float*>(kv_norm_.ptr) : nullptr,
                               eps_, cq, ctx, kv, own_);
        ctx.give(down);
        void* q = ctx.take_tokens(static_cast<long long>(H_) * D_, DType::BF16);
        ops::skinny_linear(cq, nullptr, 0.f, up_q_.weight, ctx.T, q, H_ * D_, false, nullptr, ctx.err, ctx.stream);
        ctx.give(cq);
        void* o = attend(ctx, q, kv);
        ops::skinny_linear(o, nullptr, 0.f, out_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        ctx.give(o);
    }

    // q [T, H*D] -> o [T, H*V] (a buffer the caller gives back); q is given back here
    void* attend(StepContext& ctx, void* q, KVView kv) {
        const DType act = ctx.act_dtype;
        // the key up-projection on the query's side: qa_h = W_uk,h^T q_h
        void* qa = ctx.take_tokens(static_cast<long long>(H_) * Rkv_, act);
        ops::linear_batched(q, static_cast<long long>(H_) * D_, D_, up_k_.ptr, static_cast<long long>(D_) * Rkv_, /*w_is_k_by_n=*/true, qa,
                            static_cast<long long>(H_) * Rkv_, Rkv_, act, ctx.T, Rkv_, D_, H_, ctx.stream);
        ctx.give(q);
        void* att = ctx.take_tokens(static_cast<long long>(H_) * Rkv_, act);
        kv.v_pages = kv.k_pages;
        ops::attention(ctx, qa, H_ * Rkv_, kv, att, H_, 1, Rkv_, scale_, 0);
        ctx.give(qa);
        // the value up-projection on the output's side: o_h = W_uv,h (sum_j p_j c_j)
        void* o = ctx.take_tokens(static_cast<long long>(H_) * V_, act);
        ops::linear_batched(att, static_cast<long long>(H_) * Rkv_, Rkv_, up_v_.ptr, static_cast<long long>(V_) * Rkv_, /*w_is_k_by_n=*/false, o,
                            static_cast<long long>(H_) * V_, V_, act, ctx.T, V_, Rkv_, H_, ctx.stream);
        ctx.give(att);
        return o;
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        const DType act = ctx.act_dtype;
        KVView kv = ctx.kv();
        if (kv.owns != own_)
            throw ConfigError(own_ ? "a latent-attention layer with a down-projection of its own was scheduled onto another run's cache"
                                   : "a latent-attention layer without a down-projection must read another run's cache");
        const long long down_cols = Rq_ + (own_ ? Rkv_ : 0);
        float* down = static_cast<float*>(ctx.take_tokens(down_cols, DType::F32));
        down_.apply(ctx, x, act, down, DType::F32, ctx.T, ctx.T_cap);
        void* cq = ctx.take_tokens(Rq_, act);
        ops::latent_norm_write(down, static_cast<int>(down_cols), Rq_, Rkv_, static_cast<const float*>(q_norm_.ptr),
                               own_ ? static_cast<const float*>(kv_norm_.ptr) : nullptr, eps_, cq, ctx, kv, own_);
        ctx.give(down);
        void* q = ctx.take_tokens(static_cast<long long>(H_) * D_, act);
        up_q_.apply(ctx, cq, act, q, act, ctx.T, ctx.T_cap);
        ctx.give(cq);
        void* o = attend(ctx, q, kv);
        out_.apply(ctx, o, act, out, act, ctx.T, ctx.T_cap);
        ctx.give(o);
    }

private:
    int hidden_, H_, D_, V_, Rq_, Rkv_;
    bool own_;
    float scale_, eps_;
    Linear down_, up_q_, out_;
    DeviceTensor q_norm_, kv_norm_, up_k_, up_v_;
};

namespace {
RegisterPart reg("mixer", "latent_attention", [](const json::Value& a) {
    const char* k = "latent_attention";
    return std::make_shared<LatentAttention>(static_cast<int>(arg_int(a, "hidden", k)), static_cast<int>(arg_int(a, "heads", k)),
                                             static_cast<int>(arg_int(a, "dim", k)), static_cast<int>(arg_int(a, "vdim", k)),
                                             static_cast<int>(arg_int(a, "q_rank", k)), static_cast<int>(arg_int(a, "kv_rank", k)),
                                             arg_number_or(a, "scale", 0.0, k), arg_number(a, "eps", k), arg_int_or(a, "own_latent", 1, k) != 0);
});
}  // namespace

}  // namespace vmb
