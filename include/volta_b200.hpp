// C++ host-side mirror of Volta's optimizer API over the C ABI (header only, C++17).
//
// Same type names, constructor argument order and method names as the reference:
//   volta::nn::Adam(params, lr, {beta1, beta2}, eps, weight_decay)   src/nn/optim/adam.rs:18-24
//   volta::nn::SGD(params, lr, momentum, weight_decay)               src/nn/optim/sgd.rs:28
//   volta::nn::Muon(params, lr, momentum, nesterov, ns_steps)        src/nn/optim/muon.rs:19-25
//   step(), zero_grad()                                              adam.rs:62-95, sgd.rs:58-90, muon.rs:40-163
// `Tensor` plays the role of `Rc<RefCell<RawTensor>>` (src/tensor.rs:23,38-46): shared
// ownership of {data, shape, grad: Option<..>}.  Tensors stay host resident, as Volta's CPU
// tensors are: step() uploads the gradients that are present, runs the fused device step and
// reads the parameters back (hosts that keep tensors on the device use the C ABI's
// vb_optimizer_param_ptr / vb_optimizer_grad_ptr or vb_multi_tensor_step directly).
// Where the reference panics (adam.rs:164,169,195), these classes throw std::runtime_error.
#pragma once

#include <cstdint>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "volta_b200.h"

namespace volta {

inline void vb_check(int status)
{
    if (status != VB_OK) throw std::runtime_error(std::string("volta_b200: ") + vb_last_error());
}

struct RawTensor {
    std::vector<float> data;
    std::vector<size_t> shape;
    std::optional<std::vector<float>> grad;  // `grad: Option<Storage>`
    bool requires_grad = true;

    // RawTensor::new(data, shape, requires_grad)
    static std::shared_ptr<RawTensor> make(std::vector<float> data, std::vector<size_t> shape, bool requires_grad)
    {
        size_t n = 1;
        for (size_t s : shape) n *= s;
        if (n != data.size()) throw std::runtime_error("volta_b200: shape does not match data");
        auto t = std::make_shared<RawTensor>();
        t->data = std::move(data);
        t->shape = std::move(shape);
        t->requires_grad = requires_grad;
        return t;
    }
};
using Tensor = std::shared_ptr<RawTensor>;

// One engine per process on device 0, like Volta's global GPU context (src/gpu/mod.rs:30-47).
inline vb_engine *default_engine()
{
    struct Holder {
        vb_engine *e = nullptr;
        Holder() { vb_check(vb_engine_create(0, &e)); }
        ~Holder() { vb_engine_destroy(e); }
    };
    static Holder h;
    return h.e;
}

namespace nn {

class OptimizerBase {
public:
    OptimizerBase(const OptimizerBase &) = delete;
    OptimizerBase &operator=(const OptimizerBase &) = delete;
    ~OptimizerBase() { vb_optimizer_destroy(handle_); }

    // step(): one fused update of every parameter whose gradient is present
    void step()
    {
        for (size_t i = 0; i < params_.size(); ++i) {
            RawTensor &p = *params_[i];
            if (p.grad) {
                if (p.grad->size() != p.data.size()) throw std::runtime_error("volta_b200: gradient size mismatch");
                vb_check(vb_optimizer_upload_grad(handle_, (int64_t)i, p.grad->data(), (int64_t)p.grad->size()));
            } else {
                vb_check(vb_optimizer_set_grad_present(handle_, (int64_t)i, 0));
            }
        }
        vb_check(vb_optimizer_step(handle_));
        for (size_t i = 0; i < params_.size(); ++i)
            vb_check(vb_optimizer_download_params(handle_, (int64_t)i, params_[i]->data.data(),
                                                  (int64_t)params_[i]->data.size()));
    }

    // zero_grad(): every `grad` becomes None
    void zero_grad()
    {
        for (auto &p : params_) p->grad.reset();
        vb_check(vb_optimizer_zero_grad(handle_));
    }

protected:
    explicit OptimizerBase(std::vector<Tensor> params) : params_(std::move(params)) {}
    void upload_all()
    {
        for (size_t i = 0; i < params_.size(); ++i)
            vb_check(vb_optimizer_upload_params(handle_, (int64_t)i, params_[i]->data.data(),
                                                (int64_t)params_[i]->data.size()));
    }
    std::vector<int64_t> sizes() const
    {
        std::vector<int64_t> s;
        for (auto &p : params_) s.push_back((int64_t)p->data.size());
        return s;
    }
    std::vector<Tensor> params_;
    vb_optimizer *handle_ = nullptr;
};

class Adam : public OptimizerBase {
public:
    Adam(std::vector<Tensor> params, float lr, std::pair<float, float> betas, float eps, float weight_decay)
        : OptimizerBase(std::move(params))
    {
        auto s = sizes();
        vb_check(vb_adam_create(default_engine(), (int64_t)s.size(), s.data(), lr, betas.first, betas.second, eps,
                                weight_decay, &handle_));
        upload_all();
    }
};

class SGD : public OptimizerBase {
public:
    SGD(std::vector<Tensor> params, float lr, float momentum, float weight_decay) : OptimizerBase(std::move(params))
    {
        auto s = sizes();
        vb_check(vb_sgd_create(default_engine(), (int64_t)s.size(), s.data(), lr, momentum, weight_decay, &handle_));
        upload_all();
    }
};

class Muon : public OptimizerBase {
public:
    Muon(std::vector<Tensor> params, float lr, float momentum, bool nesterov, size_t ns_steps,
         int ns_mode = VB_NS_F32)
        : OptimizerBase(std::move(params))
    {
        std::vector<int64_t> rows, cols;
        for (auto &p : params_) {  // muon.rs:117-130
            const auto &sh = p->shape;
            if (sh.size() < 2) {
                rows.push_back(sh.empty() ? 1 : (int64_t)sh[0]);
                cols.push_back(1);
            } else {
                int64_t c = 1;
                for (size_t d = 1; d < sh.size(); ++d) c *= (int64_t)sh[d];
                rows.push_back((int64_t)sh[0]);
                cols.push_back(c);
            }
        }
        vb_check(vb_muon_create(default_engine(), (int64_t)rows.size(), rows.data(), cols.data(), lr, momentum,
                                nesterov ? 1 : 0, (int)ns_steps, ns_mode, &handle_));
        upload_all();
    }
};

}  // namespace nn
}  // namespace volta
