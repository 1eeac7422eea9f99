// nnabla function-registry shim: exposes libdwbnq behind the class names nnabla-ext-cuda
// registers (DepthwiseConvolutionCuda, BatchNormalizationCuda, FixedPointQuantizeCuda,
// Pow2QuantizeCuda, MinMaxQuantizeCuda) for the backends "cuda:float" and "cuda:half", so a
// graph built with get_extension_context('cuda') dispatches to the B200 kernels unchanged.
//
// Built only against a sony/nnabla source tree (it derives from core's function classes):
//   g++ -std=c++17 -shared -fPIC -I$NNABLA_DIR/include -I<nnabla-ext-cuda>/include \
//       -I<this repo>/include dwbnq_nbla_plugin.cpp -L. -ldwbnq -lnnabla -lnnabla_cuda \
//       -o libdwbnq_nbla.so
// and loaded after nnabla_ext.cuda has been imported; dwbnq_register_nbla() then replaces
// the registry entries of the five functions (the entry registered last for a
// (function, backend) key is the one core's create_<Function>() finds first).
//
// Every forward_impl does what the reference classes do around their kernels
// (e.g. src/nbla/cuda/function/generic/depthwise_convolution.cu:435-449): make the device
// current, fetch device pointers with get_data_pointer / cast_data_and_get_pointer, launch on
// the legacy default stream, return without synchronising. A non-zero dwbnq status becomes an
// nbla::Exception through NBLA_ERROR. Backward is left to the base classes' contract:
// it raises not_implemented (this library is the inference path).
#include <dwbnq.h>

#include <nbla/cuda/common.hpp>
#include <nbla/cuda/cuda.hpp>
#include <nbla/function/batch_normalization.hpp>
#include <nbla/function/depthwise_convolution.hpp>
#include <nbla/function/fixed_point_quantize.hpp>
#include <nbla/function/min_max_quantize.hpp>
#include <nbla/function/pow2_quantize.hpp>
#include <nbla/function_registry.hpp>
#include <nbla/singleton_manager.hpp>
#include <nbla/variable.hpp>

#include <mutex>
#include <string>

namespace dwbnq_nbla {

using namespace nbla;

template <typename T> struct DType;
template <> struct DType<float> { static constexpr int value = DWBNQ_F32; };
template <> struct DType<Half> { static constexpr int value = DWBNQ_F16; };

inline void check(int status, const char *what) {
  if (status == DWBNQ_OK) return;
  const error_code code = status == DWBNQ_ERR_INVALID_ARG   ? error_code::value
                          : status == DWBNQ_ERR_UNSUPPORTED ? error_code::unclassified
                                                            : error_code::target_specific;
  NBLA_ERROR(code, "%s: %s", what, dwbnq_last_error_string());
}

#define DWBNQ_NO_BACKWARD(NAME)                                                               \
  virtual void backward_impl(const Variables &, const Variables &, const vector<bool> &,      \
                             const vector<bool> &) {                                          \
    NBLA_ERROR(error_code::not_implemented, NAME " (dwbnq) implements the forward pass only"); \
  }

// ---- DepthwiseConvolution --------------------------------------------------------------
template <typename T> class DepthwiseConvolutionCuda : public DepthwiseConvolution<T> {
public:
  typedef typename CudaType<T>::type Tc;
  explicit DepthwiseConvolutionCuda(const Context &ctx, int base_axis, const vector<int> &pad,
                                    const vector<int> &stride, const vector<int> &dilation,
                                    int multiplier)
      : DepthwiseConvolution<T>(ctx, base_axis, pad, stride, dilation, multiplier),
        device_(std::stoi(ctx.device_id)) {}
  virtual ~DepthwiseConvolutionCuda() {}
  virtual string name() { return "DepthwiseConvolutionCuda"; }
  virtual vector<string> allowed_array_classes() {
    return SingletonManager::get<Cuda>()->array_classes();
  }

protected:
  int device_;
  dwbnq_conv_desc desc_;
  virtual void setup_impl(const Variables &inputs, const Variables &outputs) {
    DepthwiseConvolution<T>::setup_impl(inputs, outputs);  // shapes, output size
    const bool two_d = this->kernel_shape_.size() == 2;
    desc_ = dwbnq_conv_desc();
    desc_.dtype = DType<T>::value;
    desc_.c = this->sample_channels_;
    desc_.n = inputs[0]->size() / inputs[0]->size(this->base_axis_);
    desc_.h = two_d ? this->sample_shape_[0] : 1;
    desc_.w = this->sample_shape_[two_d ? 1 : 0];
    desc_.kh = two_d ? this->kernel_shape_[0] : 1;
    desc_.kw = this->kernel_shape_[two_d ? 1 : 0];
    desc_.stride_h = two_d ? this->stride_[0] : 1;
    desc_.stride_w = this->stride_[two_d ? 1 : 0];
    desc_.pad_h = two_d ? this->padding_[0] : 0;
    desc_.pad_w = this->padding_[two_d ? 1 : 0];
    desc_.dil_h = two_d ? this->dilation_[0] : 1;
    desc_.dil_w = this->dilation_[two_d ? 1 : 0];
    desc_.multiplier = this->multiplier_;
    check(dwbnq_conv_out_shape(&desc_, nullptr, nullptr), "DepthwiseConvolutionCuda::setup");
  }
  virtual void forward_impl(const Variables &inputs, const Variables &outputs) {
    const Tc *x = inputs[0]->get_data_pointer<Tc>(this->ctx_);
    const Tc *w = inputs[1]->get_data_pointer<Tc>(this->ctx_);
    const Tc *b = inputs.size() == 3 ? inputs[2]->get_data_pointer<Tc>(this->ctx_) : nullptr;
    Tc *y = outputs[0]->cast_data_and_get_pointer<Tc>(this->ctx_, true);
    check(dwbnq_dwconv_fwd(&desc_, x, w, b, y, device_, nullptr), "DepthwiseConvolutionCuda::forward");
  }
  DWBNQ_NO_BACKWARD("DepthwiseConvolutionCuda")
};

// ---- BatchNormalization (batch_stat = false) ---------------------------------------------
template <typename T> class BatchNormalizationCuda : public BatchNormalization<T> {
public:
  typedef typename CudaType<T>::type Tc;
  BatchNormalizationCuda(const Context &ctx, const vector<int> axes, float decay_rate, float eps,
                         bool batch_stat, bool no_scale, bool no_bias)
      : BatchNormalization<T>(ctx, axes, decay_rate, eps, batch_stat, no_scale, no_bias),
        device_(std::stoi(ctx.device_id)) {}
  virtual ~BatchNormalizationCuda() {}
  virtual string name() { return "BatchNormalizationCuda"; }
  virtual vector<string> allowed_array_classes() {
    return SingletonManager::get<Cuda>()->array_classes();
  }

protected:
  int device_;
  virtual void forward_impl(const Variables &inputs, const Variables &outputs) {
    NBLA_CHECK(!this->batch_stat_, error_code::not_implemented,
               "BatchNormalizationCuda (dwbnq) implements batch_stat=False only");
    const Tc *x = inputs[0]->get_data_pointer<Tc>(this->ctx_);
    // (named Variable pointers: a call through inputs[<member of the dependent base>] would
    // need the `template` disambiguator)
    Variable *vb = this->no_bias_ ? nullptr : inputs[this->b_idx_];
    Variable *vg = this->no_scale_ ? nullptr : inputs[this->g_idx_];
    Variable *vm = inputs[this->m_idx_];
    Variable *vv = inputs[this->v_idx_];
    const Tc *beta = vb ? vb->get_data_pointer<Tc>(this->ctx_) : nullptr;
    const Tc *gamma = vg ? vg->get_data_pointer<Tc>(this->ctx_) : nullptr;
    const Tc *rm = vm->get_data_pointer<Tc>(this->ctx_);
    const Tc *rv = vv->get_data_pointer<Tc>(this->ctx_);
    Tc *y = outputs[0]->cast_data_and_get_pointer<Tc>(this->ctx_, true);
    check(dwbnq_bn_infer_fwd(DType<T>::value, this->size0_, this->size1_, this->size2_, this->eps_, x, beta,
                             gamma, rm, rv, y, device_, nullptr),
          "BatchNormalizationCuda::forward");
  }
  DWBNQ_NO_BACKWARD("BatchNormalizationCuda")
};

// ---- FixedPointQuantize ----------------------------------------------------------------------
template <typename T> class FixedPointQuantizeCuda : public FixedPointQuantize<T> {
public:
  typedef typename CudaType<T>::type Tc;
  explicit FixedPointQuantizeCuda(const Context &ctx, bool sign, int bw, float delta, bool ste_fine_grained)
      : FixedPointQuantize<T>(ctx, sign, bw, delta, ste_fine_grained), device_(std::stoi(ctx.device_id)) {}
  virtual ~FixedPointQuantizeCuda() {}
  virtual string name() { return "FixedPointQuantizeCuda"; }
  virtual vector<string> allowed_array_classes() {
    return SingletonManager::get<Cuda>()->array_classes();
  }

protected:
  int device_;
  virtual void forward_impl(const Variables &inputs, const Variables &outputs) {
    const Tc *x = inputs[0]->get_data_pointer<Tc>(this->ctx_);
    Tc *y = outputs[0]->cast_data_and_get_pointer<Tc>(this->ctx_, true);
    check(dwbnq_fpq_fwd(DType<T>::value, inputs[0]->size(), this->sign_, this->n_, this->delta_, x, y, device_,
                        nullptr),
          "FixedPointQuantizeCuda::forward");
  }
  DWBNQ_NO_BACKWARD("FixedPointQuantizeCuda")
};

// ---- Pow2Quantize ------------------------------------------------------------------------------
template <typename T> class Pow2QuantizeCuda : public Pow2Quantize<T> {
public:
  typedef typename CudaType<T>::type Tc;
  explicit Pow2QuantizeCuda(const Context &ctx, bool sign, bool with_zero, int n, int m, bool ste_fine_grained)
      : Pow2Quantize<T>(ctx, sign, with_zero, n, m, ste_fine_grained), device_(std::stoi(ctx.device_id)) {}
  virtual ~Pow2QuantizeCuda() {}
  virtual string name() { return "Pow2QuantizeCuda"; }
  virtual vector<string> allowed_array_classes() {
    return SingletonManager::get<Cuda>()->array_classes();
  }

protected:
  int device_;
  virtual void forward_impl(const Variables &inputs, const Variables &outputs) {
    const Tc *x = inputs[0]->get_data_pointer<Tc>(this->ctx_);
    Tc *y = outputs[0]->cast_data_and_get_pointer<Tc>(this->ctx_, true);
    check(dwbnq_pow2q_fwd(DType<T>::value, inputs[0]->size(), this->sign_, this->with_zero_, this->n_, this->m_,
                          x, y, device_, nullptr),
          "Pow2QuantizeCuda::forward");
  }
  DWBNQ_NO_BACKWARD("Pow2QuantizeCuda")
};

// ---- MinMaxQuantize (per-channel ranges [1, C, 1, 1]) --------------------------------------------
// The reference only overrides two hooks and inherits the composite from core
// (include/nbla/cuda/function/min_max_quantize.hpp:37-45); here the whole forward is one
// sequence of kernels, with the per-channel scratch held by the function object.
template <typename T> class MinMaxQuantizeCuda : public MinMaxQuantize<T> {
public:
  typedef typename CudaType<T>::type Tc;
  explicit MinMaxQuantizeCuda(const Context &ctx, float decay, bool x_min_max, bool ema, bool ste_fine_grained,
                              float eps)
      : MinMaxQuantize<T>(ctx, decay, x_min_max, ema, ste_fine_grained, eps), device_(std::stoi(ctx.device_id)) {}
  virtual ~MinMaxQuantizeCuda() {}
  virtual string name() { return "MinMaxQuantizeCuda"; }
  virtual vector<string> allowed_array_classes() {
    return SingletonManager::get<Cuda>()->array_classes();
  }

protected:
  int device_;
  Variable workspace_;
  int64_t size0_, size2_;
  int channels_;
  virtual void setup_impl(const Variables &inputs, const Variables &outputs) {
    MinMaxQuantize<T>::setup_impl(inputs, outputs);
    // ranges of shape [1, C, 1, 1]: channel axis = the one axis where qr_min is not 1
    const Shape_t xs = inputs[0]->shape(), rs = inputs[1]->shape();
    int axis = -1;
    for (size_t i = 0; i < rs.size(); ++i) {
      if (rs[i] != 1) {
        NBLA_CHECK(axis < 0 && rs[i] == xs[i], error_code::not_implemented,
                   "MinMaxQuantizeCuda (dwbnq) supports per-channel ranges along one axis");
        axis = (int)i;
      }
    }
    if (axis < 0) axis = 0;  // a single range for the whole tensor: view [1, 1, size]
    size0_ = 1;
    size2_ = 1;
    for (int i = 0; i < axis; ++i) size0_ *= xs[i];
    for (size_t i = axis + 1; i < xs.size(); ++i) size2_ *= xs[i];
    channels_ = rs.size() ? (int)rs[axis] : 1;
    if (rs.size() == 0 || rs[axis] == 1) {
      channels_ = 1;
      size0_ = 1;
      size2_ = inputs[0]->size();
    }
    workspace_.reshape(Shape_t{(Size_t)(dwbnq_workspace_bytes(channels_) / sizeof(float))}, true);
  }
  virtual void forward_impl(const Variables &inputs, const Variables &outputs) {
    dwbnq_quant_desc q = dwbnq_quant_desc();
    q.kind = DWBNQ_Q_MINMAX;
    q.decay = this->decay_;
    q.eps = this->eps_;
    q.x_min_max = this->x_min_max_;
    q.ema = this->ema_;
    dwbnq_minmax_ptrs mm;
    mm.qr_min = inputs[1]->cast_data_and_get_pointer<Tc>(this->ctx_);
    mm.qr_max = inputs[2]->cast_data_and_get_pointer<Tc>(this->ctx_);
    mm.ql_min = inputs[3]->get_data_pointer<Tc>(this->ctx_);
    mm.ql_max = inputs[4]->get_data_pointer<Tc>(this->ctx_);
    const Tc *x = inputs[0]->get_data_pointer<Tc>(this->ctx_);
    Tc *y = outputs[0]->cast_data_and_get_pointer<Tc>(this->ctx_, true);
    float *ws = workspace_.cast_data_and_get_pointer<float>(this->ctx_, true);
    check(dwbnq_minmaxq_fwd(DType<T>::value, size0_, channels_, size2_, &q, x, &mm, y, ws, nullptr, device_,
                            nullptr),
          "MinMaxQuantizeCuda::forward");
  }
  DWBNQ_NO_BACKWARD("MinMaxQuantizeCuda")
};

}  // namespace dwbnq_nbla

// Replaces the five registry entries for "cuda:float" and "cuda:half". Call once, after
// nnabla_ext.cuda (init_cuda) has registered the stock classes.
extern "C" void dwbnq_register_nbla(void) {
  using namespace nbla;
  using namespace dwbnq_nbla;
  static std::once_flag once;
  std::call_once(once, [] {
#define DWBNQ_REG(NAME, ...)                                                        \
  {                                                                                 \
    using NAME##Cuda_float = NAME##Cuda<float>;                                     \
    using NAME##Cuda_Half = NAME##Cuda<Half>;                                       \
    NBLA_REGISTER_FUNCTION_IMPL(NAME, NAME##Cuda_float, "cuda:float", __VA_ARGS__); \
    NBLA_REGISTER_FUNCTION_IMPL(NAME, NAME##Cuda_Half, "cuda:half", __VA_ARGS__);   \
  }
    DWBNQ_REG(DepthwiseConvolution, int, const vector<int> &, const vector<int> &, const vector<int> &, int)
    DWBNQ_REG(BatchNormalization, const vector<int> &, float, float, bool, bool, bool)
    DWBNQ_REG(FixedPointQuantize, bool, int, float, bool)
    DWBNQ_REG(Pow2Quantize, bool, bool, int, int, bool)
    DWBNQ_REG(MinMaxQuantize, float, bool, bool, bool, float)
#undef DWBNQ_REG
  });
}
