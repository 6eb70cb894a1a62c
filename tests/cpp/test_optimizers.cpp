// The reference's optimizer tests, replayed in C++ against the drop-in classes of
// include/volta_b200.hpp.  Each function names the reference test it follows; expected values
// are recomputed here with the same hand formulas (in float), tolerances are the reference's.
//   tests/test_optimizers.rs:13-245, tests/coverage_fill.rs:45-67, src/lib.rs:3102-3119,
//   src/nn/optim/muon.rs:172-192
#include <cmath>
#include <cstdio>
#include <functional>
#include <string>
#include <vector>

#include "volta_b200.hpp"

using volta::RawTensor;
using volta::Tensor;
using volta::nn::Adam;
using volta::nn::Muon;
using volta::nn::SGD;

static int g_failures = 0;
#define CHECK(cond, ...)                                   \
    do {                                                   \
        if (!(cond)) {                                     \
            ++g_failures;                                  \
            std::printf("  FAILED %s:%d: ", __FILE__, __LINE__); \
            std::printf(__VA_ARGS__);                      \
            std::printf("\n");                             \
        }                                                  \
    } while (0)

static float scalar(const Tensor &t) { return t->data.at(0); }
static float powi(float a, int n) { float r = 1.0f; for (int i = 0; i < n; ++i) r *= a; return r; }

static void test_adam_bias_correction()
{
    const float lr = 0.01f, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, grad_val = 0.5f, init_param = 1.0f;
    Tensor t = RawTensor::make({init_param}, {1}, true);
    t->grad = std::vector<float>{grad_val};
    Adam opt({t}, lr, {beta1, beta2}, eps, 0.0f);
    opt.step();
    const float m = (1.0f - beta1) * grad_val, v = (1.0f - beta2) * grad_val * grad_val;
    const float m_hat = m / (1.0f - beta1), v_hat = v / (1.0f - beta2);
    const float expected = init_param - lr * m_hat / (std::sqrt(v_hat) + eps);
    CHECK(std::fabs(scalar(t) - expected) < 1e-7f, "expected %.9g got %.9g", expected, scalar(t));
}

static void test_adam_mv_accumulation_multi_step()
{
    const float lr = 0.01f, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, grad_val = 0.5f;
    Tensor t = RawTensor::make({2.0f}, {1}, true);
    Adam opt({t}, lr, {beta1, beta2}, eps, 0.0f);
    float m = 0.0f, v = 0.0f, expected = 2.0f;
    for (int step = 1; step <= 3; ++step) {
        t->grad = std::vector<float>{grad_val};
        opt.step();
        m = beta1 * m + (1.0f - beta1) * grad_val;
        v = beta2 * v + (1.0f - beta2) * grad_val * grad_val;
        const float m_hat = m / (1.0f - powi(beta1, step)), v_hat = v / (1.0f - powi(beta2, step));
        expected -= lr * m_hat / (std::sqrt(v_hat) + eps);
        CHECK(std::fabs(scalar(t) - expected) < 1e-6f, "step %d expected %.9g got %.9g", step, expected, scalar(t));
    }
}

static void test_adam_weight_decay()
{
    const float lr = 0.01f, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, init_param = 2.0f;
    Tensor t_wd = RawTensor::make({init_param}, {1}, true);
    t_wd->grad = std::vector<float>{0.0f};
    Adam opt_wd({t_wd}, lr, {beta1, beta2}, eps, 0.01f);
    opt_wd.step();
    Tensor t_no = RawTensor::make({init_param}, {1}, true);
    t_no->grad = std::vector<float>{0.0f};
    Adam opt_no({t_no}, lr, {beta1, beta2}, eps, 0.0f);
    opt_no.step();
    CHECK(std::fabs(scalar(t_no) - init_param) < 1e-8f, "no-wd moved: %.9g", scalar(t_no));
    CHECK(scalar(t_wd) < init_param, "wd did not decrease the parameter");
    const float eff = 0.01f * init_param;
    const float m = (1.0f - beta1) * eff, v = (1.0f - beta2) * eff * eff;
    const float expected = init_param - lr * (m / (1.0f - beta1)) / (std::sqrt(v / (1.0f - beta2)) + eps);
    CHECK(std::fabs(scalar(t_wd) - expected) < 1e-7f, "expected %.9g got %.9g", expected, scalar(t_wd));
}

template <class Opt>
static void minimise_quadratic(Opt &opt, const Tensor &x, int steps)
{
    for (int i = 0; i < steps; ++i) {  // loss = (x - 3)^2, d/dx = 2 (x - 3)
        opt.zero_grad();
        x->grad = std::vector<float>{2.0f * (scalar(x) - 3.0f)};
        opt.step();
    }
}

static void test_adam_convergence_convex()
{
    Tensor x = RawTensor::make({0.0f}, {1}, true);
    Adam opt({x}, 0.05f, {0.9f, 0.999f}, 1e-8f, 0.0f);
    minimise_quadratic(opt, x, 500);
    CHECK(std::fabs(scalar(x) - 3.0f) < 0.05f, "got %.6g", scalar(x));
}

static void test_sgd_no_momentum_simple()
{
    Tensor t = RawTensor::make({5.0f}, {1}, true);
    t->grad = std::vector<float>{2.0f};
    SGD opt({t}, 0.1f, 0.0f, 0.0f);
    opt.step();
    const float e1 = 5.0f - 0.1f * 2.0f;
    CHECK(std::fabs(scalar(t) - e1) < 1e-7f, "expected %.9g got %.9g", e1, scalar(t));
    opt.step();  // the gradient persists across steps
    const float e2 = e1 - 0.1f * 2.0f;
    CHECK(std::fabs(scalar(t) - e2) < 1e-7f, "expected %.9g got %.9g", e2, scalar(t));
}

static void test_sgd_weight_decay()
{
    Tensor t = RawTensor::make({4.0f}, {1}, true);
    t->grad = std::vector<float>{1.0f};
    SGD opt({t}, 0.1f, 0.0f, 0.1f);
    opt.step();
    const float expected = 4.0f - 0.1f * (1.0f + 0.1f * 4.0f);
    CHECK(std::fabs(scalar(t) - expected) < 1e-7f, "expected %.9g got %.9g", expected, scalar(t));
}

static void test_sgd_convergence_convex()
{
    Tensor x = RawTensor::make({0.0f}, {1}, true);
    SGD opt({x}, 0.05f, 0.9f, 0.0f);
    minimise_quadratic(opt, x, 500);
    CHECK(std::fabs(scalar(x) - 3.0f) < 0.05f, "got %.6g", scalar(x));
}

static void test_sgd_momentum_logic()
{
    Tensor t = RawTensor::make({1.0f}, {1}, true);
    t->grad = std::vector<float>{0.1f};
    SGD opt({t}, 0.1f, 0.9f, 0.0f);
    opt.step();
    CHECK(std::fabs(scalar(t) - 0.99f) < 1e-6f, "got %.9g", scalar(t));
    opt.step();
    CHECK(std::fabs(scalar(t) - 0.971f) < 1e-6f, "got %.9g", scalar(t));
}

static void test_weight_decay_sgd()
{
    Tensor w = RawTensor::make({1.0f}, {1}, true);
    SGD opt({w}, 0.1f, 0.0f, 0.1f);
    w->grad = std::vector<float>{0.0f};
    opt.step();
    CHECK(std::fabs(scalar(w) - 0.99f) <= 1e-6f * 0.99f, "got %.9g", scalar(w));
}

static void test_muon_step()
{
    Tensor x = RawTensor::make({1.0f, -1.0f, 0.5f, 0.5f}, {2, 2}, true);
    x->grad = std::vector<float>{0.1f, 0.1f, -0.1f, -0.1f};
    Muon opt({x}, 0.1f, 0.9f, true, 5);
    const std::vector<float> before = x->data;
    opt.step();
    CHECK(before != x->data, "parameters did not change");
    for (float v : x->data) CHECK(std::fabs(v) < 2.0f, "value %.6g not below 2.0", v);
}

static void test_missing_grad_is_skipped()
{
    // adam.rs:81-84: a parameter whose grad is None keeps its value
    Tensor a = RawTensor::make({1.0f, 2.0f}, {2}, true), b = RawTensor::make({3.0f}, {1}, true);
    a->grad = std::vector<float>{0.5f, 0.5f};
    Adam opt({a, b}, 0.01f, {0.9f, 0.999f}, 1e-8f, 0.0f);
    opt.step();
    CHECK(scalar(b) == 3.0f && scalar(a) != 1.0f, "skip rule broken");
    opt.zero_grad();
    CHECK(!a->grad.has_value(), "zero_grad must drop gradients");
}

int main()
{
    const std::pair<const char *, std::function<void()>> tests[] = {
        {"test_adam_bias_correction", test_adam_bias_correction},
        {"test_adam_mv_accumulation_multi_step", test_adam_mv_accumulation_multi_step},
        {"test_adam_weight_decay", test_adam_weight_decay},
        {"test_adam_convergence_convex", test_adam_convergence_convex},
        {"test_sgd_no_momentum_simple", test_sgd_no_momentum_simple},
        {"test_sgd_weight_decay", test_sgd_weight_decay},
        {"test_sgd_convergence_convex", test_sgd_convergence_convex},
        {"test_sgd_momentum_logic", test_sgd_momentum_logic},
        {"test_weight_decay_sgd", test_weight_decay_sgd},
        {"test_muon_step", test_muon_step},
        {"test_missing_grad_is_skipped", test_missing_grad_is_skipped},
    };
    for (auto &t : tests) {
        const int before = g_failures;
        try {
            t.second();
        } catch (const std::exception &ex) {
            ++g_failures;
            std::printf("  EXCEPTION %s\n", ex.what());
        }
        std::printf("%s ... %s\n", t.first, g_failures == before ? "ok" : "FAILED");
    }
    std::printf("%d failure(s)\n", g_failures);
    return g_failures == 0 ? 0 : 1;
}
