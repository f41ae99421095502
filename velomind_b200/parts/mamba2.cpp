// The Mamba-2 state-space mixer (state-space duality), as a mixer with a fixed-size state per sequence.
//
//   W_in x = [z | x | B | C | dt]          (heads * vdim, heads * vdim, groups * state, groups * state, heads columns)
//   x, B, C pass a short causal convolution per channel (taps `conv`, with bias) and SiLU
//   dt = softplus(dt + dt_bias);  per head: S <- exp(-exp(A_log) dt) S + dt B x^T (state x vdim),  y = S^T C + D x
//   out = W_o (unit-rms over each of norm_groups equal parts of (y * silu(z)), times `norm`)
//
// What it keeps of a sequence, float32, in the cache's state area of the sequence's slot: the matrices S of all heads and the
// convolution's last conv - 1 inputs.  Both start at zero when the slot is opened and are carried from step to step.  The
// kernels are in csrc/ssm.cu; the two projections are the library's or the weight-streaming products.
#include <algorithm>

#include "args.h"
#include "linear.h"

namespace vmb {

class Mamba2 : public Mixer {
public:
    explicit Mamba2(const json::Value& a) {
        const char* k = "mamba2";
        hidden_ = static_cast<int>(arg_int(a, "hidden", k));
        H_ = static_cast<int>(arg_int(a, "heads", k));
        P_ = static_cast<int>(arg_int(a, "vdim", k));
        N_ = static_cast<int>(arg_int(a, "state", k));
        G_ = static_cast<int>(arg_int_or(a, "groups", 1, k));
        K_ = static_cast<int>(arg_int_or(a, "conv", 4, k));
        parts_ = static_cast<int>(arg_int_or(a, "norm_groups", 1, k));
        eps_ = static_cast<float>(arg_number(a, "eps", k));
        if (H_ <= 0 || P_ <= 0 || N_ <= 0 || G_ <= 0 || H_ % G_) throw ConfigError(format("part '%s': heads (%d) must be a multiple of groups (%d)", k, H_, G_));
        if (K_ < 1 || K_ > 64) throw ConfigError(format("part '%s': conv (%d) must be within 1..64", k, K_));
        if (parts_ <= 0 || (H_ * P_) % parts_) throw ConfigError(format("part '%s': norm_groups (%d) must divide heads * vdim (%d)", k, parts_, H_ * P_));
    }

    long long inner() const { return static_cast<long long>(H_) * P_; }
    long long channels() const { return inner() + 2ll * G_ * N_; }
    long long width() const { return inner() + channels() + H_; }

    WeightTable weight_specs() const override {
        WeightTable t;
        t["in"].shape = {width(), hidden_};
        t["conv"].shape = {channels(), K_};
        t["conv.b"].shape = {channels()};
        t["dt_bias"].shape = t["A_log"].shape = t["D"].shape = {H_};
        t["norm"].shape = {inner()};
        t["norm"].init_ones = true;
        t["o"].shape = {hidden_, inner()};
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        in_.bind({&w.at("in")}, bc);
        out_.bind({&w.at("o")}, bc);
        taps_ = bc.upload(w.at("conv"), DType::F32);
        conv_b_ = bc.upload(w.at("conv.b"), DType::F32);
        dt_bias_ = bc.upload(w.at("dt_bias"), DType::F32);
        A_log_ = bc.upload(w.at("A_log"), DType::F32);
        D_ = bc.upload(w.at("D"), DType::F32);
        norm_ = bc.upload(w.at("norm"), DType::F32);
    }

    bool graph_safe() const override { return true; }        // slots and token offsets are read on the device

    CacheNeed cache_need() const override {
        CacheNeed n;                                          // kind None: no keys, no values
        n.state_floats = static_cast<int>(vm_ssm_state_floats(H_, P_, N_, G_, K_));
        return n;
    }

    void mix(StepContext& ctx, const void* proj, void* y) {
        ops::ssm_mixer(proj, static_cast<int>(width()), static_cast<const float*>(taps_.ptr), static_cast<const float*>(conv_b_.ptr),
                       static_cast<const float*>(dt_bias_.ptr), static_cast<const float*>(A_log_.ptr), static_cast<const float*>(D_.ptr),
                       static_cast<const float*>(norm_.ptr), eps_, ctx, y, H_, P_, N_, G_, K_, parts_);
    }

    int max_rows() const {
        return ops::skinny_max_rows(2 * std::max(in_.weight.rows() * in_.weight.cols(), out_.weight.rows() * out_.weight.cols()));
    }

    // bfloat16: the layer's norm goes into the input projection (few tokens) and the residual sum into the output projection
    bool can_fuse(const StepContext& ctx, const Norm& norm) const override {
        const float* nw;
        float eps;
        if (!norm.as_rms(&nw, &eps) || ctx.act_dtype != DType::BF16) return false;
        if (in_.weight.dtype != DType::BF16 || out_.weight.dtype != DType::BF16) return false;
        if (hidden_ % 8 || inner() % 8 || width() % 8) return false;
        if (ctx.T_cap <= max_rows()) return hidden_ % 32 == 0 && inner() % 32 == 0;
        return true;
    }

    void forward_fused(StepContext& ctx, float* h, Norm& norm) override {
        const float* nw = nullptr;
        float eps = 0.f;
        norm.as_rms(&nw, &eps);
        const bool skinny = ctx.T_cap <= max_rows();
        void* proj = ctx.take_tokens(width(), DType::BF16);
        if (skinny && ctx.T_cap <= ops::SKINNY_NORM_ROWS) {
            ops::skinny_linear(h, nw, eps, in_.weight, ctx.T, proj, static_cast<int>(width()), false, nullptr, ctx.err, ctx.stream);
        } else {
            void* x = ctx.take_tokens(hidden_, DType::BF16);
            norm.forward(ctx, h, nullptr, x, nullptr, 0);
            if (skinny) ops::skinny_linear(x, nullptr, 0.f, in_.weight, ctx.T, proj, static_cast<int>(width()), false, nullptr, ctx.err, ctx.stream);
            else ops::linear(x, DType::BF16, hidden_, in_.weight, proj, DType::BF16, ctx.T, ctx.stream);
            ctx.give(x);
        }
        void* y = ctx.take_tokens(inner(), DType::BF16);
        mix(ctx, proj, y);
        ctx.give(proj);
        if (skinny) ops::skinny_linear(y, nullptr, 0.f, out_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        else ops::linear_residual(y, inner(), out_.weight, h, ctx.T, ctx.stream);
        ctx.give(y);
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        void* proj = ctx.take_tokens(width(), ctx.act_dtype);
        in_.apply(ctx, x, ctx.act_dtype, proj, ctx.act_dtype, ctx.T, ctx.T_cap);
        void* y = ctx.take_tokens(inner(), ctx.act_dtype);
        mix(ctx, proj, y);
        ctx.give(proj);
        out_.apply(ctx, y, ctx.act_dtype, out, ctx.act_dtype, ctx.T, ctx.T_cap);
        ctx.give(y);
    }

private:
    int hidden_ = 0, H_ = 0, P_ = 0, N_ = 0, G_ = 1, K_ = 4, parts_ = 1;
    float eps_ = 1e-6f;
    Linear in_, out_;
    DeviceTensor taps_, conv_b_, dt_bias_, A_log_, D_, norm_;
};

namespace {
RegisterPart reg("mixer", "mamba2", [](const json::Value& a) { return std::make_shared<Mamba2>(a); });
}  // namespace

}  // namespace vmb
