// TEST INFRASTRUCTURE: a minimal stand-in for the parts of nnabla core's C++ interface that
// the dwbnq registry plugin touches (nnabla itself is not installable in this environment).
// It declares the types, base-class members and macros the plugin uses, with the names the
// reference CUDA sources use for them (e.g. this->kernel_shape_, this->sample_channels_,
// this->b_idx_ in src/nbla/cuda/function/generic/{depthwise_convolution,batch_normalization}.cu),
// so that the plugin can be compiled and driven end to end by tests/test_nbla_plugin.py.
// A Variable here is a shape plus a caller-provided device pointer. Nothing of this is
// shipped; the real build uses nnabla's headers.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <tuple>
#include <type_traits>
#include <vector>

namespace nbla {
using std::shared_ptr;
using std::string;
using std::vector;
typedef int64_t Size_t;
typedef vector<int64_t> Shape_t;

struct Half { uint16_t bits; };
struct HalfCuda { uint16_t bits; };
template <typename T> struct CudaType { typedef T type; };
template <> struct CudaType<Half> { typedef HalfCuda type; };

struct Context {
  vector<string> backend;
  string array_class;
  string device_id;
};

enum class error_code { unclassified, not_implemented, value, type, memory, io, os, target_specific, target_specific_async, runtime };
class Exception : public std::runtime_error {
public:
  error_code code;
  Exception(error_code c, const string &m) : std::runtime_error(m), code(c) {}
};
inline string format_string(const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  return buf;
}
#define NBLA_ERROR(code, msg, ...) throw nbla::Exception(code, nbla::format_string(msg, ##__VA_ARGS__))
#define NBLA_CHECK(cond, code, msg, ...) \
  if (!(cond)) NBLA_ERROR(code, msg, ##__VA_ARGS__)

class Variable {
  Shape_t shape_;
  void *ptr_ = nullptr;
  void *grad_ = nullptr;  // the gradient array of the variable (caller-provided, may be null)
  std::function<void *(size_t)> alloc_;  // used by reshape() of variables the functions own

public:
  Variable() {}
  Variable(const Shape_t &s, void *p) : shape_(s), ptr_(p) {}
  static std::function<void *(size_t)> &default_alloc() {
    static std::function<void *(size_t)> f;
    return f;
  }
  Shape_t shape() const { return shape_; }
  Size_t size(int axis = -1) const {
    Size_t n = 1;
    for (size_t i = axis < 0 ? 0 : (size_t)axis; i < shape_.size(); ++i) n *= shape_[i];
    return n;
  }
  // a Variable that wraps a caller's buffer keeps it; one a function owns gets scratch
  void reshape(const Shape_t &s, bool) {
    shape_ = s;
    if (!ptr_) ptr_ = default_alloc()((size_t)size() * sizeof(float));
  }
  void set_grad(void *g) { grad_ = g; }
  template <typename T> const T *get_grad_pointer(const Context &) { return static_cast<const T *>(grad_); }
  template <typename T> T *cast_grad_and_get_pointer(const Context &, bool = false) { return static_cast<T *>(grad_); }
  template <typename T> const T *get_data_pointer(const Context &) { return static_cast<const T *>(ptr_); }
  template <typename T> T *cast_data_and_get_pointer(const Context &, bool = false) { return static_cast<T *>(ptr_); }
};
typedef vector<Variable *> Variables;

class Cuda {
public:
  vector<string> array_classes() const { return {"CudaCachedArray", "CudaArray"}; }
};
struct SingletonManager {
  template <typename S> static S *get() {
    static S s;
    return &s;
  }
};

enum class dtypes { FLOAT, HALF };
template <typename T> dtypes get_dtype() { return std::is_same<T, Half>::value ? dtypes::HALF : dtypes::FLOAT; }

class Function {
protected:
  Context ctx_;

public:
  explicit Function(const Context &ctx) : ctx_(ctx) {}
  virtual ~Function() {}
  virtual string name() = 0;
  virtual vector<string> allowed_array_classes() = 0;
  // supplied by the generated base class of a core function; a function without one (the
  // plugin's fused layer) defines them itself
  virtual shared_ptr<Function> copy() const { return nullptr; }
  virtual vector<dtypes> in_types() { return {}; }
  virtual vector<dtypes> out_types() { return {}; }
  virtual int min_inputs() { return 0; }
  virtual int min_outputs() { return 0; }
  void setup(const Variables &i, const Variables &o) { setup_impl(i, o); }
  void forward(const Variables &i, const Variables &o) { forward_impl(i, o); }
  void backward(const Variables &i, const Variables &o, const vector<bool> &p, const vector<bool> &a) {
    backward_impl(i, o, p, a);
  }

protected:
  virtual void setup_impl(const Variables &, const Variables &) = 0;
  virtual void forward_impl(const Variables &, const Variables &) = 0;
  virtual void backward_impl(const Variables &, const Variables &, const vector<bool> &, const vector<bool> &) = 0;
};

// Base of every function class: keeps the constructor arguments (core: nbla/function.hpp).
template <typename... Args> class BaseFunction : public Function {
protected:
  std::tuple<typename std::remove_cv<typename std::remove_reference<Args>::type>::type...> args_;

public:
  BaseFunction(const Context &ctx, Args... args) : Function(ctx), args_(args...) {}
  int num_args() const { return (int)sizeof...(Args); }
};

// ---- the five base functions: constructor arguments and the members the CUDA classes read --
template <typename T> class DepthwiseConvolution : public Function {
protected:
  int base_axis_;
  vector<int> padding_, stride_, dilation_;
  int multiplier_;
  vector<int> sample_shape_, outmap_shape_, kernel_shape_;
  int sample_channels_, outmap_channels_;

public:
  DepthwiseConvolution(const Context &ctx, int base_axis, const vector<int> &pad, const vector<int> &stride,
                       const vector<int> &dilation, int multiplier)
      : Function(ctx), base_axis_(base_axis), padding_(pad), stride_(stride), dilation_(dilation),
        multiplier_(multiplier) {}

protected:
  virtual void setup_impl(const Variables &inputs, const Variables &) {
    const Shape_t xs = inputs[0]->shape(), ws = inputs[1]->shape();
    sample_channels_ = (int)xs[base_axis_];
    outmap_channels_ = sample_channels_ * multiplier_;
    sample_shape_.clear();
    kernel_shape_.clear();
    outmap_shape_.clear();
    for (size_t i = base_axis_ + 1; i < xs.size(); ++i) sample_shape_.push_back((int)xs[i]);
    for (size_t i = 1; i < ws.size(); ++i) kernel_shape_.push_back((int)ws[i]);
    for (size_t i = 0; i < kernel_shape_.size(); ++i)
      outmap_shape_.push_back((sample_shape_[i] + 2 * padding_[i] - dilation_[i] * (kernel_shape_[i] - 1) - 1) /
                                  stride_[i] + 1);
  }
};

template <typename T> class BatchNormalization : public Function {
protected:
  vector<int> axes_;
  float decay_rate_, eps_;
  bool batch_stat_, no_scale_, no_bias_;
  int b_idx_, g_idx_, m_idx_, v_idx_;
  Size_t size0_, size1_, size2_;

public:
  BatchNormalization(const Context &ctx, const vector<int> axes, float decay_rate, float eps, bool batch_stat,
                     bool no_scale, bool no_bias)
      : Function(ctx), axes_(axes), decay_rate_(decay_rate), eps_(eps), batch_stat_(batch_stat),
        no_scale_(no_scale), no_bias_(no_bias) {}

protected:
  virtual void setup_impl(const Variables &inputs, const Variables &) {
    // inputs: x, [beta], [gamma], mean, var
    b_idx_ = no_bias_ ? -1 : 1;
    g_idx_ = no_scale_ ? -1 : (no_bias_ ? 1 : 2);
    m_idx_ = 1 + (no_bias_ ? 0 : 1) + (no_scale_ ? 0 : 1);
    v_idx_ = m_idx_ + 1;
    const Shape_t xs = inputs[0]->shape();
    const int ax = axes_[0];
    size0_ = 1;
    size2_ = 1;
    for (int i = 0; i < ax; ++i) size0_ *= xs[i];
    size1_ = xs[ax];
    for (size_t i = ax + 1; i < xs.size(); ++i) size2_ *= xs[i];
  }
};

template <typename T> class FixedPointQuantize : public Function {
protected:
  bool sign_;
  int n_;
  float delta_;
  bool ste_fine_grained_;
  float max_, min_;

public:
  FixedPointQuantize(const Context &ctx, bool sign, int n, float delta, bool ste)
      : Function(ctx), sign_(sign), n_(n), delta_(delta), ste_fine_grained_(ste) {}

protected:
  virtual void setup_impl(const Variables &, const Variables &) {}
};

template <typename T> class Pow2Quantize : public Function {
protected:
  bool sign_, with_zero_;
  int n_, m_;
  bool ste_fine_grained_;
  float p_max_, p_min_, pruning_threshold_;

public:
  Pow2Quantize(const Context &ctx, bool sign, bool with_zero, int n, int m, bool ste)
      : Function(ctx), sign_(sign), with_zero_(with_zero), n_(n), m_(m), ste_fine_grained_(ste) {}

protected:
  virtual void setup_impl(const Variables &, const Variables &) {}
};

template <typename T> class MinMaxQuantize : public Function {
protected:
  float decay_;
  bool x_min_max_, ema_, ste_fine_grained_;
  float eps_;

public:
  MinMaxQuantize(const Context &ctx, float decay, bool x_min_max, bool ema, bool ste, float eps)
      : Function(ctx), decay_(decay), x_min_max_(x_min_max), ema_(ema), ste_fine_grained_(ste), eps_(eps) {}

protected:
  virtual void setup_impl(const Variables &, const Variables &) {}
};

// ---- registry: (function name, backend) -> factory, later registrations win ----------------
struct StubRegistry {
  static std::map<string, std::shared_ptr<void>> &table() {
    static std::map<string, std::shared_ptr<void>> t;
    return t;
  }
};
template <typename Impl, typename... Args> struct StubFactory {
  std::function<Function *(const Context &, Args...)> make = [](const Context &c, Args... a) -> Function * {
    return new Impl(c, a...);
  };
};
#define NBLA_REGISTER_FUNCTION_IMPL(BASE, CLS, BACKEND, ...)                                    \
  nbla::StubRegistry::table()[std::string(#BASE) + "/" + BACKEND] =                             \
      std::static_pointer_cast<void>(std::make_shared<nbla::StubFactory<CLS, ##__VA_ARGS__>>())

template <typename... Args>
Function *stub_create(const string &base, const string &backend, const Context &ctx, Args... args) {
  auto it = StubRegistry::table().find(base + "/" + backend);
  if (it == StubRegistry::table().end()) NBLA_ERROR(error_code::unclassified, "%s not registered for %s", base.c_str(), backend.c_str());
  typedef std::function<Function *(const Context &, Args...)> Fn;
  // every factory starts with its std::function member
  return (*reinterpret_cast<Fn *>(it->second.get()))(ctx, args...);
}
}  // namespace nbla
