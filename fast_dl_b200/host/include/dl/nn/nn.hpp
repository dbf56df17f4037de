// dl::nn -- forward-only modules (fast_dl has no autograd).  Module, Linear, ReLU and
// Sequential behave as in include/dl/nn/*.hpp: Linear holds weight [in, out] and a zero bias
// [out], initialised Kaiming- or Xavier-uniform from a process-wide seed counter that starts
// at 1234 (src/nn/Linear.cpp:10-13); Sequential owns its modules and registers them as
// children; parameters() walks registered children in order.
#pragma once

#include <memory>
#include <vector>

#include <dl/tensor/Tensor.hpp>

namespace dl::nn {

class Module {
public:
    virtual ~Module() = default;
    virtual Tensor forward(const Tensor& input) = 0;

    /// Parameters of all registered children, depth-first in registration order.
    virtual std::vector<Tensor*> parameters() {
        std::vector<Tensor*> all;
        for (Module* child : children_) {
            for (Tensor* p : child->parameters()) all.push_back(p);
        }
        return all;
    }

    Tensor operator()(const Tensor& input) { return forward(input); }

protected:
    /// Non-owning: the child must outlive this module.
    void register_module(Module& child) { children_.push_back(&child); }

private:
    std::vector<Module*> children_;
};

enum class LinearInit { XavierUniform, KaimingUniform };

class Linear : public Module {
public:
    Linear(int in_features, int out_features, const Device& device,
           LinearInit init = LinearInit::KaimingUniform);
    Tensor forward(const Tensor& input) override;
    std::vector<Tensor*> parameters() override;

private:
    Tensor weight_;
    Tensor bias_;
};

class ReLU : public Module {
public:
    Tensor forward(const Tensor& input) override;
};

class Sequential : public Module {
public:
    void add(std::unique_ptr<Module> module);
    Tensor forward(const Tensor& input) override;

private:
    std::vector<std::unique_ptr<Module>> modules_;
};

}  // namespace dl::nn
