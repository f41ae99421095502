// The mLSTM layer of xLSTM as a mixer: a matrix memory per head and sequence instead of keys and values.
//
// What it keeps of a sequence is a fixed-size float32 state (per head S [dim, vdim], n [dim] and the running maximum m of the
// log gates), held in the cache's state area of the sequence's slot; it starts at zero when the slot is opened and is
// carried from step to step.  The recurrence, the soft-capped gates and the output stage (unit norm per head, learned scale,
// sigmoid gate) are in csrc/mlstm.cu; here: one stacked projection (q | k | v | g | input gate | forget gate) with a
// float32 result, the recurrence, the output projection.
#include <algorithm>

#include "args.h"
#include "linear.h"

namespace vmb {

class MatrixLSTM : public Mixer {
public:
    MatrixLSTM(int hidden, int heads, int dim, int vdim, double gate_cap, double eps)
        : hidden_(hidden), H_(heads), D_(dim), V_(vdim), cap_(static_cast<float>(gate_cap)), eps_(static_cast<float>(eps)) {
        if (!(gate_cap > 0)) throw ConfigError("part 'mlstm': gate_cap must be positive");
    }

    WeightTable weight_specs() const override {
        WeightTable t;
        t["q"].shape = t["k"].shape = {static_cast<long long>(H_) * D_, hidden_};
        t["v"].shape = t["g"].shape = {static_cast<long long>(H_) * V_, hidden_};
        t["i"].shape = t["f"].shape = {H_, hidden_};
        t["i.b"].shape = t["f.b"].shape = {H_};
        t["norm"].shape = {static_cast<long long>(H_) * V_};
        t["norm"].init_ones = true;
        t["o"].shape = {hidden_, static_cast<long long>(H_) * V_};
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        proj_.bind({&w.at("q"), &w.at("k"), &w.at("v"), &w.at("g"), &w.at("i"), &w.at("f")}, bc);
        bias_i_ = bc.upload(w.at("i.b"), DType::F32);
        bias_f_ = bc.upload(w.at("f.b"), DType::F32);
        norm_ = bc.upload(w.at("norm"), DType::F32);
        out_.bind({&w.at("o")}, bc);
    }

    bool graph_safe() const override { return true; }        // slots and token offsets are read on the device

    CacheNeed cache_need() const override {
        CacheNeed n;                                          // kind None: no keys, no values
        n.state_floats = H_ * (D_ * V_ + D_ + 1);
        return n;
    }

    // Few tokens (decode steps) in bfloat16: the weight-streaming products, the layer's norm taken into the stacked projection
    // and the residual sum into the output projection.
    bool can_fuse(const StepContext& ctx, const Norm& norm) const override {
        const float* nw;
        float eps;
        if (!norm.as_rms(&nw, &eps) || ctx.act_dtype != DType::BF16) return false;
        if (proj_.weight.dtype != DType::BF16 || out_.weight.dtype != DType::BF16) return false;
        const long long most = std::max(proj_.weight.rows() * proj_.weight.cols(), out_.weight.rows() * out_.weight.cols());
        if (ctx.T_cap > std::min(ops::skinny_max_rows(2 * most), ops::SKINNY_NORM_ROWS)) return false;
        return hidden_ % 32 == 0 && (H_ * V_) % 32 == 0 && proj_.weight.rows() % 8 == 0;
    }

    void forward_fused(StepContext& ctx, float* h, Norm& norm) override {
        const float* nw = nullptr;
        float eps = 0.f;
        norm.as_rms(&nw, &eps);
        const int cols = static_cast<int>(proj_.weight.rows());
        float* proj = static_cast<float*>(ctx.take_tokens(cols, DType::F32));
        ops::skinny_linear(h, nw, eps, proj_.weight, ctx.T, proj, cols, true, nullptr, ctx.err, ctx.stream);
        void* y = ctx.take_tokens(static_cast<long long>(H_) * V_, DType::BF16);
        ops::mlstm_scan(proj, cols, static_cast<const float*>(bias_i_.ptr), static_cast<const float*>(bias_f_.ptr), static_cast<const float*>(norm_.ptr),
                        ctx, y, H_, D_, V_, cap_, eps_);
        ctx.give(proj);
        ops::skinny_linear(y, nullptr, 0.f, out_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        ctx.give(y);
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        const long long cols = 2ll * H_ * D_ + 2ll * H_ * V_ + 2ll * H_;
        float* proj = static_cast<float*>(ctx.take_tokens(cols, DType::F32));
        proj_.apply(ctx, x, ctx.act_dtype, proj, DType::F32, ctx.T, ctx.T_cap);
        void* y = ctx.take_tokens(static_cast<long long>(H_) * V_, ctx.act_dtype);
        ops::mlstm_scan(proj, static_cast<int>(cols), static_cast<const float*>(bias_i_.ptr), static_cast<const float*>(bias_f_.ptr),
                        static_cast<const float*>(norm_.ptr), ctx, y, H_, D_, V_, cap_, eps_);
        ctx.give(proj);
        out_.apply(ctx, y, ctx.act_dtype, out, ctx.act_dtype, ctx.T, ctx.T_cap);
        ctx.give(y);
    }

private:
    int hidden_, H_, D_, V_;
    float cap_, eps_;
    Linear proj_, out_;
    DeviceTensor bias_i_, bias_f_, norm_;
};

namespace {
RegisterPart reg("mixer", "mlstm", [](const json::Value& a) {
    const char* k = "mlstm";
    return std::make_shared<MatrixLSTM>(static_cast<int>(arg_int(a, "hidden", k)), static_cast<int>(arg_int(a, "heads", k)),
                                        static_cast<int>(arg_int(a, "dim", k)), static_cast<int>(arg_int(a, "vdim", k)), arg_number(a, "gate_cap", k),
                                        arg_number(a, "eps", k));
});
}  // namespace

}  // namespace vmb
