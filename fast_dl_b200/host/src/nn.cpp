// Forward-only modules.
#include <dl/nn/nn.hpp>

#include <dl/ops/Ops.hpp>

#include <stdexcept>
#include <utility>

namespace dl::nn {

namespace {
// One counter for the whole process, first value 1234: two Linear layers built in the same
// order get the same weights in every run.
uint64_t next_init_seed() {
    static uint64_t next = 1234;
    return next++;
}
}  // namespace

Linear::Linear(int in_features, int out_features, const Device& device, LinearInit init) {
    if (in_features <= 0 || out_features <= 0) throw std::runtime_error("Linear features must be positive");
    const Shape wshape({in_features, out_features});
    const uint64_t seed = next_init_seed();
    weight_ = init == LinearInit::XavierUniform ? Tensor::xavier_uniform(wshape, DType::Float32, device, seed)
                                                 : Tensor::kaiming_uniform(wshape, DType::Float32, device, seed);
    bias_ = Tensor::zeros(Shape({out_features}), DType::Float32, device);
}

Tensor Linear::forward(const Tensor& input) { return ops::linear(input, weight_, bias_); }
std::vector<Tensor*> Linear::parameters() { return {&weight_, &bias_}; }

Tensor ReLU::forward(const Tensor& input) { return ops::relu(input); }

void Sequential::add(std::unique_ptr<Module> module) {
    if (!module) throw std::runtime_error("Sequential cannot add a null module");
    modules_.push_back(std::move(module));
    register_module(*modules_.back());
}

Tensor Sequential::forward(const Tensor& input) {
    Tensor x = input;
    for (auto& m : modules_) x = m->forward(x);
    return x;
}

}  // namespace dl::nn
