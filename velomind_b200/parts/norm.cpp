// Root-mean-square norm with a learned scale.
#include "args.h"
#include "../engine/ops.h"

namespace vmb {

// y = x / sqrt(mean(x^2) + eps) * weight, statistics in float32 (src/cpu/ops/rmsnorm.cpp:42-59).  The residual add that
// precedes a norm in a pre-norm block is fused into the same kernel.
class RMSNorm : public Norm {
public:
    // `tensor`: what the scale is called behind the part's prefix ("weight" unless the checkpoint says otherwise; may be empty)
    RMSNorm(int size, float eps, std::string tensor = "weight") : size_(size), eps_(eps), tensor_(std::move(tensor)) {}
    WeightTable weight_specs() const override {
        WeightSpec s;
        s.shape = {size_};
        s.init_ones = true;
        return {{tensor_, s}};
    }
    void bind(const Weights& w, BindContext& bc) override { weight_ = bc.upload(w.at(tensor_), DType::F32); }   // exact for BF16 and F32 storage
    bool graph_safe() const override { return true; }
    bool as_rms(const float** weight, float* eps) const override {
        *weight = static_cast<const float*>(weight_.ptr);
        *eps = eps_;
        return true;
    }
    void forward(StepContext& ctx, float* h, const void* delta, void* out, const int* rows, int n_rows) override {
        ops::add_rmsnorm(h, delta, static_cast<const float*>(weight_.ptr), eps_, out, rows, rows ? n_rows : ctx.T, size_, ctx.act_dtype, ctx.stream);
    }

private:
    int size_;
    float eps_;
    std::string tensor_;
    DeviceTensor weight_;
};

namespace {
RegisterPart reg("norm", "rmsnorm", [](const json::Value& a) {
    return std::make_shared<RMSNorm>(static_cast<int>(arg_int(a, "size", "rmsnorm")), static_cast<float>(arg_number(a, "eps", "rmsnorm")),
                                     arg_string_or(a, "tensor", "weight", "rmsnorm"));
});

// The norm of a layer half that does not exist (a layer without a feed-forward): no weights, never run.
class NoNorm : public Norm {
public:
    bool graph_safe() const override { return true; }
    void forward(StepContext&, float*, const void*, void*, const int*, int) override { throw Error("a norm of kind 'none' stands for a part that is not there; it cannot run"); }
};
RegisterPart reg_none("norm", "none", [](const json::Value&) { return std::make_shared<NoNorm>(); });
}  // namespace

}  // namespace vmb
