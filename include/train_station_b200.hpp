// C++17 host mirror of the reference's Rust API over the C ABI of train_station_b200.h: the same type and method
// names (Tensor::matmul / add_tensor / relu / pow_scalar / sum / mean / backward / grad_by_value, NoGradTrack,
// Adam::add_parameter / step / zero_grad), the same argument meaning, and an exception where the reference panics or
// returns Err.  Header-only; link against libtrain_station_b200.so.  A compiled host has none of an interpreter's
// per-call cost, which is what bounds the small, launch-latency-bound configurations.
//
// Reference interfaces mirrored (paths inside the train-station crate):
//   tensor/core/mod.rs, tensor/init/basic.rs, tensor/init/data.rs        Tensor, constructors, from_slice
//   tensor/ops/*.rs, tensor/reductions/*.rs, tensor/transform/*.rs       the operations
//   tensor/core/operators.rs                                             + - * / between tensors and with f32
//   gradtrack/engine.rs, gradtrack/no_grad_track.rs                      backward, clear_gradients, NoGradTrack
//   optimizers/adam/mod.rs                                               AdamConfig, Adam
#pragma once

#include <cstddef>
#include <initializer_list>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "train_station_b200.h"

namespace train_station {

// What a panic or an Err of the reference becomes: the message is the library's last error text.
class Error : public std::runtime_error {
public:
    explicit Error(const std::string& what) : std::runtime_error(what) {}
};

namespace detail {
inline std::string last_error(const char* what) {
    const char* e = ts_last_error();
    return (e && *e) ? std::string(e) : std::string(what) + " failed";
}
inline void require(bool ok, const char* what) {
    if (!ok) throw Error(last_error(what));
}
inline std::vector<unsigned long long> ull(const std::vector<size_t>& v) { return std::vector<unsigned long long>(v.begin(), v.end()); }
}  // namespace detail

// shape.rs: the dims of a tensor (strides are implied: a transposed / permuted view keeps its axis order internally)
struct Shape {
    std::vector<size_t> dims;
    size_t rank() const { return dims.size(); }
    size_t size() const {
        size_t n = 1;
        for (size_t d : dims) n *= d;
        return n;
    }
    bool operator==(const Shape& o) const { return dims == o.dims; }
};

// device/mod.rs cuda_is_available / cuda_device_count / set_default_device over cuda_wrapper.h:14-16
inline int cuda_device_count() { return get_cuda_device_count(); }
inline bool cuda_is_available() { return get_cuda_device_count() > 0; }
inline void set_default_device(int index) { detail::require(set_cuda_device(index) && cuda_ffi_initialize(), "set_default_device"); }
inline void synchronize() { detail::require(ts_sync_stream(nullptr), "synchronize"); }
enum class MatmulPrecision { FP32 = 0, TF32 = 1, TF32x3 = 2 };
inline void set_matmul_precision(MatmulPrecision p) { detail::require(ts_set_matmul_precision(static_cast<int>(p)), "set_matmul_precision"); }

class Tensor {
public:
    Tensor() = default;   // an empty handle; every method on it throws

    // ---- constructors (tensor/init/basic.rs:52-215, tensor/init/data.rs:71-111, tensor/init/random.rs:66-130)
    static Tensor new_(const std::vector<size_t>& dims) { auto d = detail::ull(dims); return wrap(ts_tensor_new(d.data(), (int)d.size()), "Tensor::new"); }
    static Tensor zeros(const std::vector<size_t>& dims) { auto d = detail::ull(dims); return wrap(ts_tensor_zeros(d.data(), (int)d.size()), "Tensor::zeros"); }
    static Tensor ones(const std::vector<size_t>& dims) { auto d = detail::ull(dims); return wrap(ts_tensor_ones(d.data(), (int)d.size()), "Tensor::ones"); }
    static Tensor from_slice(const float* data, size_t len, const std::vector<size_t>& dims) {
        size_t n = 1;
        for (size_t d : dims) n *= d;
        if (n != len) throw Error("Data size " + std::to_string(len) + " doesn't match shape size " + std::to_string(n));   // data.rs:88-95
        auto d = detail::ull(dims);
        return wrap(ts_tensor_from_slice(data, d.data(), (int)d.size()), "Tensor::from_slice");
    }
    static Tensor from_slice(const std::vector<float>& data, const std::vector<size_t>& dims) { return from_slice(data.data(), data.size(), dims); }
    static Tensor randn(const std::vector<size_t>& dims, std::optional<unsigned long long> seed = std::nullopt) {
        auto d = detail::ull(dims);
        return wrap(ts_tensor_randn(d.data(), (int)d.size(), seed.value_or(0), seed.has_value()), "Tensor::randn");
    }

    // ---- properties
    bool defined() const { return static_cast<bool>(h_); }
    unsigned long long id() const { return ts_tensor_id(get()); }
    size_t size() const { return ts_tensor_size(get()); }
    Shape shape() const {
        std::vector<unsigned long long> d((size_t)ts_tensor_rank(get()));
        detail::require(d.empty() || ts_tensor_dims(get(), d.data()), "shape");
        return Shape{std::vector<size_t>(d.begin(), d.end())};
    }
    bool requires_grad() const { return ts_tensor_requires_grad(get()); }
    Tensor with_requires_grad() && { set_requires_grad(true); return std::move(*this); }
    Tensor with_requires_grad() const& { Tensor t = *this; t.set_requires_grad(true); return t; }
    void set_requires_grad(bool flag) { detail::require(ts_tensor_set_requires_grad(get(), flag), "set_requires_grad"); }
    // the device address of the elements (materialises a deferred result)
    float* data_ptr() const { float* p = ts_tensor_data_ptr(get()); detail::require(p || size() == 0, "data_ptr"); return p; }
    // a host copy of the elements (the reference's data() borrows; a device tensor has to copy)
    std::vector<float> data() const {
        std::vector<float> out(size());
        detail::require(out.empty() || ts_tensor_to_host(get(), out.data()), "data");
        return out;
    }
    float value() const {       // core/utils.rs: only a one-element tensor has a value
        if (size() != 1) throw Error("value() can only be called on tensors with exactly one element");
        return data()[0];
    }
    void copy_from_host(const float* host) { detail::require(ts_tensor_copy_from_host(get(), host), "copy_from_host"); }
    void fill(float v) { detail::require(ts_tensor_fill(get(), v), "fill"); }

    // ---- the path: matmul, the four binary ops (NumPy-style broadcasting), relu, pow_scalar, sum, mean
    Tensor matmul(const Tensor& o) const { return wrap(ts_tensor_matmul(get(), o.get()), "matmul"); }
    Tensor add_tensor(const Tensor& o) const { return wrap(ts_tensor_add_tensor(get(), o.get()), "add_tensor"); }
    Tensor sub_tensor(const Tensor& o) const { return wrap(ts_tensor_sub_tensor(get(), o.get()), "sub_tensor"); }
    Tensor mul_tensor(const Tensor& o) const { return wrap(ts_tensor_mul_tensor(get(), o.get()), "mul_tensor"); }
    Tensor div_tensor(const Tensor& o) const { return wrap(ts_tensor_div_tensor(get(), o.get()), "div_tensor"); }
    Tensor relu() const { return wrap(ts_tensor_relu(get()), "relu"); }
    Tensor pow_scalar(float e) const { return wrap(ts_tensor_pow_scalar(get(), e), "pow_scalar"); }
    Tensor sum() const { return wrap(ts_tensor_sum(get()), "sum"); }
    Tensor mean() const { return wrap(ts_tensor_mean(get()), "mean"); }

    // ---- the other elementwise ops
    Tensor exp() const { return wrap(ts_tensor_exp(get()), "exp"); }
    Tensor log() const { return wrap(ts_tensor_log(get()), "log"); }
    Tensor sqrt() const { return wrap(ts_tensor_sqrt(get()), "sqrt"); }
    Tensor tanh() const { return wrap(ts_tensor_tanh(get()), "tanh"); }
    Tensor sigmoid() const { return wrap(ts_tensor_sigmoid(get()), "sigmoid"); }
    Tensor leaky_relu(float negative_slope) const { return wrap(ts_tensor_leaky_relu(get(), negative_slope), "leaky_relu"); }
    Tensor softmax(size_t dim) const { return wrap(ts_tensor_softmax(get(), dim), "softmax"); }
    Tensor add_scalar(float s) const { return wrap(ts_tensor_add_scalar(get(), s), "add_scalar"); }
    Tensor sub_scalar(float s) const { return wrap(ts_tensor_sub_scalar(get(), s), "sub_scalar"); }
    Tensor mul_scalar(float s) const { return wrap(ts_tensor_mul_scalar(get(), s), "mul_scalar"); }
    Tensor div_scalar(float s) const { return wrap(ts_tensor_div_scalar(get(), s), "div_scalar"); }

    // ---- reductions over axes (tensor/reductions/*.rs): kinds follow enum ts_reduce_kind
    Tensor sum_dims(const std::vector<size_t>& dims, bool keepdim) const { return reduce_dims(0, dims, keepdim, "sum_dims"); }
    Tensor mean_dims(const std::vector<size_t>& dims, bool keepdim) const { return reduce_dims(1, dims, keepdim, "mean_dims"); }
    Tensor max_dims(const std::vector<size_t>& dims, bool keepdim) const { return reduce_dims(2, dims, keepdim, "max_dims"); }
    Tensor min_dims(const std::vector<size_t>& dims, bool keepdim) const { return reduce_dims(3, dims, keepdim, "min_dims"); }
    Tensor norm_dims(const std::vector<size_t>& dims, bool keepdim) const { return reduce_dims(4, dims, keepdim, "norm_dims"); }
    Tensor var_dims(const std::vector<size_t>& dims, bool keepdim) const { return reduce_dims(5, dims, keepdim, "var_dims"); }
    Tensor std_dims(const std::vector<size_t>& dims, bool keepdim) const { return reduce_dims(6, dims, keepdim, "std_dims"); }
    Tensor max() const { return wrap(ts_tensor_reduce_all(get(), 2), "max"); }
    Tensor min() const { return wrap(ts_tensor_reduce_all(get(), 3), "min"); }
    Tensor norm() const { return wrap(ts_tensor_reduce_all(get(), 4), "norm"); }
    Tensor var() const { return wrap(ts_tensor_reduce_all(get(), 5), "var"); }
    Tensor std() const { return wrap(ts_tensor_reduce_all(get(), 6), "std"); }

    // ---- layout (tensor/transform/*.rs)
    Tensor reshape(const std::vector<long long>& new_shape) const { return wrap(ts_tensor_reshape(get(), new_shape.data(), (int)new_shape.size()), "reshape"); }
    Tensor view(const std::vector<long long>& new_shape) const { return reshape(new_shape); }
    Tensor flatten() const { return reshape({-1}); }
    Tensor transpose(size_t dim0, size_t dim1) const { return wrap(ts_tensor_transpose(get(), dim0, dim1), "transpose"); }
    Tensor t() const {
        if (shape().rank() != 2) throw Error("Matrix transpose requires 2D tensor");   // transpose.rs:283-291
        return transpose(0, 1);
    }
    Tensor permute(const std::vector<size_t>& order) const { auto o = detail::ull(order); return wrap(ts_tensor_permute(get(), o.data(), (int)o.size()), "permute"); }
    Tensor contiguous() const { return wrap(ts_tensor_contiguous(get()), "contiguous"); }
    // false for the views transpose / t / permute return: they share this tensor's storage (transpose.rs:181-184)
    bool is_contiguous() const { return ts_tensor_is_contiguous(get()); }
    Tensor clone() const { return wrap(ts_tensor_clone(get()), "clone"); }
    static Tensor cat(const std::vector<Tensor>& tensors, size_t dim) {
        std::vector<ts_tensor*> hs;
        for (const Tensor& t : tensors) hs.push_back(t.get());
        return wrap(ts_tensor_cat(hs.data(), (int)hs.size(), dim), "cat");
    }

    // ---- gradtrack (gradtrack/engine.rs): backward from this tensor, the gradient of a leaf by value
    void backward(const std::optional<Tensor>& grad_output = std::nullopt) const {
        detail::require(ts_tensor_backward(get(), grad_output ? grad_output->get() : nullptr), "backward");
    }
    std::optional<Tensor> grad_by_value() const {
        ts_tensor* g = ts_tensor_grad_by_value(get());
        if (!g) return std::nullopt;
        return Tensor(g);
    }

    ts_tensor* get() const {
        if (!h_) throw Error("use of an empty Tensor handle");
        return h_.get();
    }

private:
    explicit Tensor(ts_tensor* h) : h_(h, ts_tensor_free) {}
    static Tensor wrap(ts_tensor* h, const char* what) {
        if (!h) throw Error(detail::last_error(what));
        return Tensor(h);
    }
    Tensor reduce_dims(int kind, const std::vector<size_t>& dims, bool keepdim, const char* what) const {
        auto d = detail::ull(dims);
        return wrap(ts_tensor_reduce_dims(get(), kind, d.data(), (int)d.size(), keepdim), what);
    }
    std::shared_ptr<ts_tensor> h_;
    friend class Adam;
};

// tensor/core/operators.rs: tensor-tensor forms forward to *_tensor, tensor-scalar forms to *_scalar
inline Tensor operator+(const Tensor& a, const Tensor& b) { return a.add_tensor(b); }
inline Tensor operator-(const Tensor& a, const Tensor& b) { return a.sub_tensor(b); }
inline Tensor operator*(const Tensor& a, const Tensor& b) { return a.mul_tensor(b); }
inline Tensor operator/(const Tensor& a, const Tensor& b) { return a.div_tensor(b); }
inline Tensor operator+(const Tensor& a, float s) { return a.add_scalar(s); }
inline Tensor operator-(const Tensor& a, float s) { return a.sub_scalar(s); }
inline Tensor operator*(const Tensor& a, float s) { return a.mul_scalar(s); }
inline Tensor operator/(const Tensor& a, float s) { return a.div_scalar(s); }
inline Tensor operator+(float s, const Tensor& a) { return a.add_scalar(s); }
inline Tensor operator*(float s, const Tensor& a) { return a.mul_scalar(s); }
inline Tensor operator-(const Tensor& a) { return a.mul_scalar(-1.0f); }

// gradtrack/engine.rs:812-816
inline void clear_gradients() { ts_clear_gradients(); }
inline bool is_grad_enabled() { return ts_is_grad_enabled(); }

// gradtrack/no_grad_track.rs: gradient tracking is off while one of these lives
class NoGradTrack {
public:
    NoGradTrack() { ts_no_grad_push(); }
    ~NoGradTrack() { ts_no_grad_pop(); }
    NoGradTrack(const NoGradTrack&) = delete;
    NoGradTrack& operator=(const NoGradTrack&) = delete;
};

// optimizers/adam/mod.rs:111-155: the defaults are the reference's (and PyTorch's)
struct AdamConfig {
    float learning_rate = 1e-3f;
    float beta1 = 0.9f;
    float beta2 = 0.999f;
    float eps = 1e-8f;
    float weight_decay = 0.0f;
    bool amsgrad = false;
};

// optimizers/adam/mod.rs:180-560.  Parameters are linked by tensor id; step() takes the parameters in any order,
// skips (with a message, as the reference prints) those without a gradient and fails for an unlinked one.
class Adam {
public:
    Adam() : Adam(AdamConfig{}) {}
    explicit Adam(const AdamConfig& c) : config_(c), h_(ts_adam_new_amsgrad(c.learning_rate, c.beta1, c.beta2, c.eps, c.weight_decay, c.amsgrad), ts_adam_free) {
        if (!h_) throw Error(detail::last_error("Adam::new"));
    }
    static Adam new_() { return Adam(); }
    static Adam with_config(const AdamConfig& c) { return Adam(c); }
    static Adam with_learning_rate(float lr) {
        AdamConfig c;
        c.learning_rate = lr;
        return Adam(c);
    }
    void add_parameter(const Tensor& p) { detail::require(ts_adam_add_parameter(h_.get(), p.get()), "Adam::add_parameter"); }
    void add_parameters(const std::vector<const Tensor*>& ps) { for (const Tensor* p : ps) add_parameter(*p); }
    void step(const std::vector<Tensor*>& params) {
        handles(params);
        detail::require(ts_adam_step(h_.get(), scratch_.data(), (int)scratch_.size(), 1.0f), "Adam::step");
    }
    void zero_grad(const std::vector<Tensor*>& params) {
        handles(params);
        ts_adam_zero_grad(h_.get(), scratch_.data(), (int)scratch_.size());
    }
    float learning_rate() const { return ts_adam_learning_rate(h_.get()); }
    void set_learning_rate(float lr) { ts_adam_set_learning_rate(h_.get(), lr); }
    unsigned long long step_count() const { return ts_adam_step_count(h_.get()); }
    const AdamConfig& config() const { return config_; }
    // the moment estimates of a linked parameter (first, second), as copies of the handles the optimizer holds
    std::pair<Tensor, Tensor> state(const Tensor& p) const {
        return {Tensor::wrap(ts_adam_state_m(h_.get(), p.get()), "Adam::state"), Tensor::wrap(ts_adam_state_v(h_.get(), p.get()), "Adam::state")};
    }

private:
    void handles(const std::vector<Tensor*>& params) {
        scratch_.clear();
        for (Tensor* p : params) scratch_.push_back(p->get());
    }
    AdamConfig config_;
    std::shared_ptr<ts_adam> h_;
    std::vector<ts_tensor*> scratch_;
};

}  // namespace train_station
