// A routed feed-forward (mixture of experts) with an optional shared expert.
//
//   z = W_router x + b (float32)          the `top` experts with the largest logits are chosen
//   w = softmax over the chosen logits    y = sum_k w_k W_down[e_k] act(W_up[e_k] x)
//   shared expert (if any): runs for every token and is added, times sigmoid(w_sg . x) if it has a gate
//
// Experts are two-layer networks without biases; `activation` names theirs (the shared expert may have another).  The router,
// its bias and the shared gate stay float32 on the device whatever the compute dtype.
#include "args.h"
#include "linear.h"

namespace vmb {

int activation_code(const std::string& name, const char* part) {
    if (name == "silu") return VM_ACT_SILU;
    if (name == "gelu_tanh") return VM_ACT_GELU_TANH;
    if (name == "relu_squared") return VM_ACT_RELU_SQUARED;
    throw ConfigError(format("part '%s': activation '%s' is not known (silu, gelu_tanh, relu_squared)", part, name.c_str()));
}

class RoutedExperts : public FeedForward {
public:
    RoutedExperts(int hidden, int experts, int top, int ff, int act, int shared_ff, int shared_act, bool shared_gate)
        : hidden_(hidden), E_(experts), top_(top), ff_(ff), act_(act), sff_(shared_ff), sact_(shared_act), gate_(shared_gate && shared_ff > 0) {
        if (top < 1 || top > experts) throw ConfigError(format("part 'routed_experts': top (%d) must be within 1..experts (%d)", top, experts));
    }

    WeightTable weight_specs() const override {
        WeightTable t;
        t["router"].shape = {E_, hidden_};
        t["router.b"].shape = {E_};
        for (int e = 0; e < E_; ++e) {
            t[format("e%d.up", e)].shape = {ff_, hidden_};
            t[format("e%d.down", e)].shape = {hidden_, ff_};
        }
        if (sff_ > 0) {
            t["shared.up"].shape = {sff_, hidden_};
            t["shared.down"].shape = {hidden_, sff_};
            if (gate_) t["shared.sg"].shape = {1, hidden_};
        }
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        router_ = bc.upload(w.at("router"), DType::F32);
        router_b_ = bc.upload(w.at("router.b"), DType::F32);
        std::vector<const HostTensor*> ups, downs, all;
        for (int e = 0; e < E_; ++e) {
            ups.push_back(&w.at(format("e%d.up", e)));
            downs.push_back(&w.at(format("e%d.down", e)));
        }
        all = ups;
        all.insert(all.end(), downs.begin(), downs.end());
        if (sff_ > 0) {
            all.push_back(&w.at("shared.up"));
            all.push_back(&w.at("shared.down"));
        }
        const DType kept = bc.matrix_dtype(all);           // one dtype for every expert matrix
        up_ = bc.upload_stacked(ups, kept);
        down_ = bc.upload_stacked(downs, kept);
        if (sff_ > 0) {
            s_up_ = bc.upload(w.at("shared.up"), kept);
            s_down_ = bc.upload(w.at("shared.down"), kept);
            if (gate_) s_gate_ = bc.upload(w.at("shared.sg"), DType::F32);
        }
    }

    bool graph_safe() const override { return true; }

    // whether a step of this capacity groups its pairs by expert (many tokens) or streams each token's experts (few)
    bool grouped(const StepContext& ctx) const {
        return ctx.act_dtype == DType::BF16 && up_.dtype == DType::BF16 && hidden_ % 32 == 0 && ff_ % 32 == 0 && ctx.T_cap > GROUPED_FROM_TOKENS &&
               !ctx.one_token_each;
    }

    // Few tokens in bfloat16: router and up-projections norm the residual stream's rows themselves, the down-projections add
    // into it: three launches for the layer half.
    bool can_fuse(const StepContext& ctx, const Norm& norm) const override {
        const float* nw;
        float eps;
        return norm.as_rms(&nw, &eps) && ctx.act_dtype == DType::BF16 && !grouped(ctx);
    }

    void forward_fused(StepContext& ctx, float* h, Norm& norm) override {
        const float* nw = nullptr;
        float eps = 0.f;
        norm.as_rms(&nw, &eps);
        run_few(ctx, h, nw, eps, nullptr, h);
    }

    // the few-token path: x in the activation dtype, or (nw given) the float32 residual stream; `residual` given: added into
    void run_few(StepContext& ctx, const void* x, const float* nw, float eps, void* out, float* residual) {
        int* chosen = static_cast<int*>(ctx.take_tokens(top_, DType::I32));
        float* weight = static_cast<float*>(ctx.take_tokens(top_, DType::F32));
        float* sgate = gate_ ? static_cast<float*>(ctx.take_tokens(1, DType::F32)) : nullptr;
        ops::expert_router(x, nw, eps, static_cast<const float*>(router_.ptr), static_cast<const float*>(router_b_.ptr),
                           gate_ ? static_cast<const float*>(s_gate_.ptr) : nullptr, ctx.T, hidden_, E_, top_, chosen, weight, sgate, ctx.act_dtype,
                           ctx.stream);
        void* act = ctx.take_tokens(static_cast<long long>(top_) * ff_ + sff_, ctx.act_dtype);
        ops::experts_few_tokens(x, nw, eps, up_, down_, sff_ > 0 ? s_up_.ptr : nullptr, sff_ > 0 ? s_down_.ptr : nullptr, chosen, weight, sgate, ctx.T,
                                hidden_, ff_, sff_, top_, act_, sact_, act, out, residual, ctx.act_dtype, ctx.stream);
        ctx.give(act);
        ctx.give(sgate);
        ctx.give(weight);
        ctx.give(chosen);
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        if (!grouped(ctx)) {
            run_few(ctx, x, nullptr, 0.f, out, nullptr);
            return;
        }
        int* chosen = static_cast<int*>(ctx.take_tokens(top_, DType::I32));
        float* weight = static_cast<float*>(ctx.take_tokens(top_, DType::F32));
        float* sgate = gate_ ? static_cast<float*>(ctx.take_tokens(1, DType::F32)) : nullptr;
        ops::expert_router(x, nullptr, 0.f, static_cast<const float*>(router_.ptr), static_cast<const float*>(router_b_.ptr),
                           gate_ ? static_cast<const float*>(s_gate_.ptr) : nullptr, ctx.T, hidden_, E_, top_, chosen, weight, sgate, ctx.act_dtype,
                           ctx.stream);
        // Many tokens (by the step's capacity, so that a bucket's steps ask for the same scratch): pairs grouped by expert, tensor-core
        // tiles per expert, the shared expert as two library products.  Few tokens: every token streams the rows of its experts.
        {
            float* shared_y = nullptr;
            if (sff_ > 0) {
                void* u = ctx.take_tokens(sff_, DType::BF16);
                ops::linear(x, DType::BF16, hidden_, s_up_, u, DType::BF16, ctx.T, ctx.stream);
                ops::activation(u, u, static_cast<long long>(ctx.T) * sff_, sact_, DType::BF16, ctx.stream);
                shared_y = static_cast<float*>(ctx.take_tokens(hidden_, DType::F32));
                ops::linear(u, DType::BF16, sff_, s_down_, shared_y, DType::F32, ctx.T, ctx.stream);
                ctx.give(u);
            }
            // the experts' tiles on tcgen05 from TC_FROM_TOKENS on (tiles of 128 rows, rows gathered first), on mma.sync below
            const bool tc = ctx.T_cap >= TC_FROM_TOKENS && ctx.err != nullptr;
            const int row_cap = static_cast<int>(tc ? vm_experts_grouped_rows_tiled(ctx.T_cap, top_, E_, 128) : vm_experts_grouped_rows(ctx.T_cap, top_, E_));
            int* row_of_pair = static_cast<int*>(ctx.take_tokens(top_, DType::I32));
            int* token_of_row = static_cast<int*>(ctx.take(row_cap, DType::I32));
            int* expert_of_tile = static_cast<int*>(ctx.take(row_cap / 64, DType::I32));
            void* act = ctx.take(static_cast<long long>(row_cap) * ff_, DType::BF16);
            float* y = static_cast<float*>(ctx.take(static_cast<long long>(row_cap) * hidden_, DType::F32));
            if (tc) {
                void* x_sorted = ctx.take(static_cast<long long>(row_cap) * hidden_, DType::BF16);
                ops::experts_grouped_tc(x, up_, down_, chosen, weight, shared_y, sgate, ctx.T, hidden_, ff_, top_, E_, act_, row_cap, row_of_pair,
                                        token_of_row, expert_of_tile, x_sorted, act, y, out, ctx.err, ctx.stream);
                ctx.give(x_sorted);
            } else {
                ops::experts_grouped(x, up_, down_, chosen, weight, shared_y, sgate, ctx.T, hidden_, ff_, top_, E_, act_, row_cap, row_of_pair,
                                     token_of_row, expert_of_tile, act, y, out, ctx.stream);
            }
            ctx.give(y);
            ctx.give(act);
            ctx.give(expert_of_tile);
            ctx.give(token_of_row);
            ctx.give(row_of_pair);
            ctx.give(shared_y);
            ctx.give(sgate);
            ctx.give(weight);
            ctx.give(chosen);
            return;
        }
    }

    static constexpr int GROUPED_FROM_TOKENS = 64;      // a step's capacity above which the pairs are grouped by expert
    static constexpr int TC_FROM_TOKENS = 256;          // ... and from which the experts' tiles run on tcgen05

private:
    int hidden_, E_, top_, ff_, act_, sff_, sact_;
    bool gate_;
    DeviceTensor router_, router_b_, up_, down_, s_up_, s_down_, s_gate_;
};

namespace {
RegisterPart reg("feed_forward", "routed_experts", [](const json::Value& a) {
    const char* k = "routed_experts";
    const std::string act = arg_string_or(a, "activation", "relu_squared", k);
    return std::make_shared<RoutedExperts>(static_cast<int>(arg_int(a, "hidden", k)), static_cast<int>(arg_int(a, "experts", k)),
                                           static_cast<int>(arg_int(a, "top", k)), static_cast<int>(arg_int(a, "ff", k)), activation_code(act, k),
                                           static_cast<int>(arg_int_or(a, "shared_ff", 0, k)),
                                           activation_code(arg_string_or(a, "shared_activation", act, k), k), arg_int_or(a, "shared_gate", 1, k) != 0);
});
}  // namespace

}  // namespace vmb
