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
// nbla::Exception through NBLA_ERROR. Backward: DepthwiseConvolution (float), FixedPointQuantize
// and Pow2Quantize call the library's backward entry points with the reference's
// propagate_down / accum semantics; BatchNormalization, MinMaxQuantize and the fused function
// object raise not_implemented (inference path).
//
// Besides the five registered classes the plugin holds FusedDwBnQuantCuda, the single
// function object a graph converter substitutes for a whole dw-conv -> BN -> quantizer
// chain, and its factory dwbnq_nbla_create_fused(); and FusedPwBnQuantCuda with
// dwbnq_nbla_create_fused_pw() for the pointwise convolution -> BN -> activation -> quantizer
// chains either side of it.
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
  // The reference's backward_impl (depthwise_convolution.cu:492-650): a gradient is computed
  // when its propagate_down flag is set and overwritten unless its accum flag is set.
  virtual void backward_impl(const Variables &inputs, const Variables &outputs, const vector<bool> &propagate_down,
                             const vector<bool> &accum) {
    const bool has_bias = inputs.size() == 3;
    if (!(propagate_down[0] || propagate_down[1] || (has_bias && propagate_down[2]))) return;
    const Tc *x = inputs[0]->get_data_pointer<Tc>(this->ctx_);
    const Tc *w = inputs[1]->get_data_pointer<Tc>(this->ctx_);
    const Tc *dy = outputs[0]->get_grad_pointer<Tc>(this->ctx_);
    Tc *dx = propagate_down[0] ? inputs[0]->cast_grad_and_get_pointer<Tc>(this->ctx_, !accum[0]) : nullptr;
    Tc *dw = propagate_down[1] ? inputs[1]->cast_grad_and_get_pointer<Tc>(this->ctx_, !accum[1]) : nullptr;
    Tc *db = (has_bias && propagate_down[2]) ? inputs[2]->cast_grad_and_get_pointer<Tc>(this->ctx_, !accum[2]) : nullptr;
    const int mask = (accum[0] ? 1 : 0) | (accum[1] ? 2 : 0) | ((has_bias && accum[2]) ? 4 : 0);
    check(dwbnq_dwconv_bwd(&desc_, x, w, dy, dx, dw, db, mask, device_, nullptr), "DepthwiseConvolutionCuda::backward");
  }
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
  virtual void backward_impl(const Variables &inputs, const Variables &outputs, const vector<bool> &propagate_down,
                             const vector<bool> &accum) {
    if (!propagate_down[0]) return;
    Tc *dx = inputs[0]->cast_grad_and_get_pointer<Tc>(this->ctx_, !accum[0]);
    const Tc *dy = outputs[0]->get_grad_pointer<Tc>(this->ctx_);
    const Tc *x = inputs[0]->get_data_pointer<Tc>(this->ctx_);
    check(dwbnq_fpq_bwd(DType<T>::value, inputs[0]->size(), this->sign_, this->n_, this->delta_,
                        this->ste_fine_grained_, accum[0], x, dy, dx, device_, nullptr),
          "FixedPointQuantizeCuda::backward");
  }
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
  virtual void backward_impl(const Variables &inputs, const Variables &outputs, const vector<bool> &propagate_down,
                             const vector<bool> &accum) {
    if (!propagate_down[0]) return;
    const Tc *x = inputs[0]->get_data_pointer<Tc>(this->ctx_);
    Tc *dx = inputs[0]->cast_grad_and_get_pointer<Tc>(this->ctx_, !accum[0]);
    const Tc *dy = outputs[0]->get_grad_pointer<Tc>(this->ctx_);
    check(dwbnq_pow2q_bwd(DType<T>::value, inputs[0]->size(), this->sign_, this->with_zero_, this->n_, this->m_,
                          this->ste_fine_grained_, accum[0], x, dy, dx, device_, nullptr),
          "Pow2QuantizeCuda::backward");
  }
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

// ---- the fused layer: DepthwiseConvolution -> BatchNormalization(batch_stat=false) -> quantizer --
// One function object for the three-function chain, which is what a graph converter puts in
// the chain's place (the way nnabla's BatchNormalizationFolding replaces conv -> BN by one
// convolution): its constructor takes the constructor arguments of the three functions it
// replaces, its inputs are theirs in order,
//   [x, w, (b), (beta), (gamma), mean, var, (qr_min, qr_max, ql_min, ql_max)]
// (b when with_bias; beta / gamma unless no_bias / no_scale; the four range tensors for
// MinMaxQuantize), and its one output is the quantizer's. forward_impl is one call of
// dwbnq_fused_fwd: x is read once and the quantized y written once, instead of three
// kernels with two intermediate tensors. It derives from core's BaseFunction like every
// generated function class (include/nbla/cuda/function/function_impl.hpp.tmpl:29-58 shows
// the shape of a derived CUDA class); there is no core base class for it, so the members a
// generated base would supply (copy, in/out types, min inputs/outputs, output shape) are here.
template <typename T>
class FusedDwBnQuantCuda
    : public BaseFunction<int, const vector<int> &, const vector<int> &, const vector<int> &, int, bool,
                          float, bool, bool, int, bool, bool, int, int, float, float, bool, bool, float> {
public:
  typedef typename CudaType<T>::type Tc;
  typedef BaseFunction<int, const vector<int> &, const vector<int> &, const vector<int> &, int, bool, float,
                       bool, bool, int, bool, bool, int, int, float, float, bool, bool, float>
      Base;
  // conv: base_axis, pad, stride, dilation, multiplier (+ whether a bias input is present);
  // BN: eps, no_scale, no_bias (axes = [base_axis], batch_stat = false by construction);
  // quantizer: kind (dwbnq_quant_kind) and the union of the three quantizers' arguments.
  FusedDwBnQuantCuda(const Context &ctx, int base_axis, const vector<int> &pad, const vector<int> &stride,
                     const vector<int> &dilation, int multiplier, bool with_bias, float bn_eps, bool no_scale,
                     bool no_bias, int quant_kind, bool sign, bool with_zero, int n, int m, float delta,
                     float decay, bool x_min_max, bool ema, float mm_eps)
      : Base(ctx, base_axis, pad, stride, dilation, multiplier, with_bias, bn_eps, no_scale, no_bias, quant_kind,
             sign, with_zero, n, m, delta, decay, x_min_max, ema, mm_eps),
        base_axis_(base_axis), pad_(pad), stride_(stride), dilation_(dilation), multiplier_(multiplier),
        with_bias_(with_bias), bn_eps_(bn_eps), no_scale_(no_scale), no_bias_(no_bias),
        device_(std::stoi(ctx.device_id)) {
    q_ = dwbnq_quant_desc();
    q_.kind = quant_kind;
    q_.sign = sign;
    q_.with_zero = with_zero;
    q_.n = n;
    q_.m = m;
    q_.delta = delta;
    q_.decay = decay;
    q_.x_min_max = x_min_max;
    q_.ema = ema;
    q_.eps = mm_eps;
  }
  virtual ~FusedDwBnQuantCuda() {}
  virtual shared_ptr<Function> copy() const {
    return shared_ptr<Function>(new FusedDwBnQuantCuda<T>(
        this->ctx_, base_axis_, pad_, stride_, dilation_, multiplier_, with_bias_, bn_eps_, no_scale_, no_bias_,
        q_.kind, q_.sign != 0, q_.with_zero != 0, q_.n, q_.m, q_.delta, q_.decay, q_.x_min_max != 0, q_.ema != 0,
        q_.eps));
  }
  virtual vector<dtypes> in_types() { return vector<dtypes>(n_inputs(), get_dtype<T>()); }
  virtual vector<dtypes> out_types() { return vector<dtypes>{get_dtype<T>()}; }
  virtual int min_inputs() { return n_inputs(); }
  virtual int min_outputs() { return 1; }
  virtual string name() { return "FusedDwBnQuantCuda"; }
  virtual vector<string> allowed_array_classes() {
    return SingletonManager::get<Cuda>()->array_classes();
  }

protected:
  int base_axis_;
  vector<int> pad_, stride_, dilation_;
  int multiplier_;
  bool with_bias_;
  float bn_eps_;
  bool no_scale_, no_bias_;
  int device_;
  dwbnq_quant_desc q_;
  dwbnq_conv_desc desc_;
  Variable workspace_;
  int n_inputs() const {
    return 2 + (with_bias_ ? 1 : 0) + (no_bias_ ? 0 : 1) + (no_scale_ ? 0 : 1) + 2 +
           (q_.kind == DWBNQ_Q_MINMAX ? 4 : 0);
  }
  virtual void setup_impl(const Variables &inputs, const Variables &outputs) {
    NBLA_CHECK((int)inputs.size() == n_inputs(), error_code::value,
               "FusedDwBnQuantCuda expects %d inputs, got %d", n_inputs(), (int)inputs.size());
    const Shape_t xs = inputs[0]->shape(), ws = inputs[1]->shape();
    const int sdims = (int)xs.size() - base_axis_ - 1;
    NBLA_CHECK(sdims == 1 || sdims == 2, error_code::value, "1-D or 2-D depthwise convolution expected");
    NBLA_CHECK((int)ws.size() == sdims + 1 && (int)pad_.size() == sdims && (int)stride_.size() == sdims &&
                   (int)dilation_.size() == sdims,
               error_code::value, "weight rank / pad / stride / dilation do not match %d spatial dims", sdims);
    const bool two_d = sdims == 2;
    desc_ = dwbnq_conv_desc();
    desc_.dtype = DType<T>::value;
    desc_.c = (int)xs[base_axis_];
    desc_.n = 1;
    for (int i = 0; i < base_axis_; ++i) desc_.n *= xs[i];
    desc_.h = two_d ? (int)xs[base_axis_ + 1] : 1;
    desc_.w = (int)xs[base_axis_ + (two_d ? 2 : 1)];
    desc_.kh = two_d ? (int)ws[1] : 1;
    desc_.kw = (int)ws[two_d ? 2 : 1];
    desc_.stride_h = two_d ? stride_[0] : 1;
    desc_.stride_w = stride_[two_d ? 1 : 0];
    desc_.pad_h = two_d ? pad_[0] : 0;
    desc_.pad_w = pad_[two_d ? 1 : 0];
    desc_.dil_h = two_d ? dilation_[0] : 1;
    desc_.dil_w = dilation_[two_d ? 1 : 0];
    desc_.multiplier = multiplier_;
    NBLA_CHECK(ws[0] == (Size_t)desc_.c * multiplier_, error_code::value,
               "weight has %d output maps, expected channels x multiplier = %d", (int)ws[0], desc_.c * multiplier_);
    int32_t ho = 0, wo = 0;
    check(dwbnq_conv_out_shape(&desc_, &ho, &wo), "FusedDwBnQuantCuda::setup");
    Shape_t ys(xs.begin(), xs.begin() + base_axis_);
    ys.push_back(ws[0]);
    if (two_d) ys.push_back(ho);
    ys.push_back(wo);
    outputs[0]->reshape(ys, true);
    if (q_.kind == DWBNQ_Q_MINMAX)
      workspace_.reshape(Shape_t{(Size_t)(dwbnq_workspace_bytes((int)ws[0]) / sizeof(float))}, true);
  }
  virtual void forward_impl(const Variables &inputs, const Variables &outputs) {
    int i = 0;
    const Tc *x = inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    const Tc *w = inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    const Tc *b = with_bias_ ? inputs[i++]->get_data_pointer<Tc>(this->ctx_) : nullptr;
    const Tc *beta = no_bias_ ? nullptr : inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    const Tc *gamma = no_scale_ ? nullptr : inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    const Tc *rm = inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    const Tc *rv = inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    dwbnq_minmax_ptrs mm = dwbnq_minmax_ptrs();
    float *ws = nullptr;
    if (q_.kind == DWBNQ_Q_MINMAX) {
      mm.qr_min = inputs[i++]->cast_data_and_get_pointer<Tc>(this->ctx_);
      mm.qr_max = inputs[i++]->cast_data_and_get_pointer<Tc>(this->ctx_);
      mm.ql_min = inputs[i++]->get_data_pointer<Tc>(this->ctx_);
      mm.ql_max = inputs[i++]->get_data_pointer<Tc>(this->ctx_);
      ws = workspace_.cast_data_and_get_pointer<float>(this->ctx_, true);
    }
    Tc *y = outputs[0]->cast_data_and_get_pointer<Tc>(this->ctx_, true);
    check(dwbnq_fused_fwd(&desc_, bn_eps_, &q_, x, w, b, beta, gamma, rm, rv,
                          q_.kind == DWBNQ_Q_MINMAX ? &mm : nullptr, y, ws, nullptr, device_, nullptr),
          "FusedDwBnQuantCuda::forward");
  }
  DWBNQ_NO_BACKWARD("FusedDwBnQuantCuda")
};

// ---- the pointwise chain ------------------------------------------------------------------
// Convolution (1x1, pad 0, stride 1, dilation 1, group 1) -> BatchNormalization
// (batch_stat = false) -> [ReLU | ReLU6] -> FixedPointQuantize | Pow2Quantize as one function
// object, the counterpart of FusedDwBnQuantCuda for the convolutions either side of a depthwise
// layer. Inputs [x, w, (b), (beta), (gamma), mean, var], one output. The accuracy mode of the
// sum follows the switch the reference has for its GEMMs: three TF32 passes (fp32 class)
// unless TF32 is allowed (NNABLA_CUDA_ALLOW_TF32, src/nbla/cuda/init.cpp.tmpl:76-83).
template <typename T>
class FusedPwBnQuantCuda
    : public BaseFunction<int, bool, float, bool, bool, int, int, bool, bool, int, int, float, bool> {
public:
  typedef typename CudaType<T>::type Tc;
  typedef BaseFunction<int, bool, float, bool, bool, int, int, bool, bool, int, int, float, bool> Base;
  FusedPwBnQuantCuda(const Context &ctx, int base_axis, bool with_bias, float bn_eps, bool no_scale, bool no_bias,
                     int act, int quant_kind, bool sign, bool with_zero, int n, int m, float delta, bool allow_tf32)
      : Base(ctx, base_axis, with_bias, bn_eps, no_scale, no_bias, act, quant_kind, sign, with_zero, n, m, delta,
             allow_tf32),
        base_axis_(base_axis), with_bias_(with_bias), bn_eps_(bn_eps), no_scale_(no_scale), no_bias_(no_bias),
        act_(act), allow_tf32_(allow_tf32), device_(std::stoi(ctx.device_id)) {
    q_ = dwbnq_quant_desc();
    q_.kind = quant_kind;
    q_.sign = sign;
    q_.with_zero = with_zero;
    q_.n = n;
    q_.m = m;
    q_.delta = delta;
  }
  virtual ~FusedPwBnQuantCuda() {}
  virtual shared_ptr<Function> copy() const {
    return shared_ptr<Function>(new FusedPwBnQuantCuda<T>(this->ctx_, base_axis_, with_bias_, bn_eps_, no_scale_,
                                                          no_bias_, act_, q_.kind, q_.sign != 0, q_.with_zero != 0,
                                                          q_.n, q_.m, q_.delta, allow_tf32_));
  }
  virtual vector<dtypes> in_types() { return vector<dtypes>(n_inputs(), get_dtype<T>()); }
  virtual vector<dtypes> out_types() { return vector<dtypes>{get_dtype<T>()}; }
  virtual int min_inputs() { return n_inputs(); }
  virtual int min_outputs() { return 1; }
  virtual string name() { return "FusedPwBnQuantCuda"; }
  virtual vector<string> allowed_array_classes() { return SingletonManager::get<Cuda>()->array_classes(); }

protected:
  int base_axis_;
  bool with_bias_;
  float bn_eps_;
  bool no_scale_, no_bias_;
  int act_;
  bool allow_tf32_;
  int device_;
  dwbnq_quant_desc q_;
  dwbnq_pwconv_desc desc_;
  Variable workspace_;
  int n_inputs() const { return 2 + (with_bias_ ? 1 : 0) + (no_bias_ ? 0 : 1) + (no_scale_ ? 0 : 1) + 2; }
  virtual void setup_impl(const Variables &inputs, const Variables &outputs) {
    NBLA_CHECK((int)inputs.size() == n_inputs(), error_code::value, "FusedPwBnQuantCuda expects %d inputs, got %d",
               n_inputs(), (int)inputs.size());
    const Shape_t xs = inputs[0]->shape(), ws = inputs[1]->shape();
    NBLA_CHECK((int)xs.size() == base_axis_ + 3, error_code::value, "a 2-D convolution input [.., c_in, h, w] is expected");
    NBLA_CHECK(ws.size() == 4 && ws[2] == 1 && ws[3] == 1 && ws[1] == xs[base_axis_], error_code::value,
               "the weight must be [c_out, c_in, 1, 1] over the input's %d channels", (int)xs[base_axis_]);
    desc_ = dwbnq_pwconv_desc();
    desc_.dtype = DType<T>::value;
    desc_.c_in = (int)ws[1];
    desc_.c_out = (int)ws[0];
    desc_.h = (int)xs[base_axis_ + 1];
    desc_.w = (int)xs[base_axis_ + 2];
    desc_.n = 1;
    for (int i = 0; i < base_axis_; ++i) desc_.n *= xs[i];
    desc_.math = allow_tf32_ ? DWBNQ_PW_MATH_TF32 : DWBNQ_PW_MATH_FP32;
    desc_.act = act_;
    const size_t bytes = dwbnq_pwconv_workspace_bytes(&desc_);
    if (bytes == 0) check(DWBNQ_ERR_INVALID_ARG, "FusedPwBnQuantCuda::setup");
    Shape_t ys(xs.begin(), xs.begin() + base_axis_);
    ys.push_back(ws[0]);
    ys.push_back(xs[base_axis_ + 1]);
    ys.push_back(xs[base_axis_ + 2]);
    outputs[0]->reshape(ys, true);
    workspace_.reshape(Shape_t{(Size_t)(bytes / sizeof(float))}, true);
  }
  virtual void forward_impl(const Variables &inputs, const Variables &outputs) {
    int i = 0;
    const Tc *x = inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    const Tc *w = inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    const Tc *b = with_bias_ ? inputs[i++]->get_data_pointer<Tc>(this->ctx_) : nullptr;
    const Tc *beta = no_bias_ ? nullptr : inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    const Tc *gamma = no_scale_ ? nullptr : inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    const Tc *rm = inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    const Tc *rv = inputs[i++]->get_data_pointer<Tc>(this->ctx_);
    Tc *y = outputs[0]->cast_data_and_get_pointer<Tc>(this->ctx_, true);
    float *ws = workspace_.cast_data_and_get_pointer<float>(this->ctx_, true);
    check(dwbnq_pwconv_fused_fwd(&desc_, bn_eps_, &q_, x, w, b, beta, gamma, rm, rv, y, ws, device_, nullptr),
          "FusedPwBnQuantCuda::forward");
  }
  DWBNQ_NO_BACKWARD("FusedPwBnQuantCuda")
};

}  // namespace dwbnq_nbla

// Factory of the fused function object, for the graph converter that replaces a matched
// DepthwiseConvolution -> BatchNormalization -> quantizer chain (INTEGRATION.md shows the
// converter). Arguments are plain C values: the constructor arguments of the three
// functions; pad / stride / dilation point to `spatial_dims` ints each. `half` selects the
// "cuda:half" class. Returns a new nbla::Function* (the caller wraps it in a FunctionPtr /
// CgFunction, which then owns it), or NULL with the reason in dwbnq_last_error_string()
// when an argument is out of range.
extern "C" void *dwbnq_nbla_create_fused(int half, int device, int base_axis, int spatial_dims, const int *pad,
                                         const int *stride, const int *dilation, int multiplier, int with_bias,
                                         float bn_eps, int no_scale, int no_bias, int quant_kind, int sign,
                                         int with_zero, int n, int m, float delta, float decay, int x_min_max,
                                         int ema, float mm_eps) {
  using namespace nbla;
  using namespace dwbnq_nbla;
  if (spatial_dims < 1 || spatial_dims > 2 || !pad || !stride || !dilation || quant_kind < DWBNQ_Q_NONE ||
      quant_kind > DWBNQ_Q_MINMAX || base_axis < 0 || device < 0)
    return nullptr;
  Context ctx;
  ctx.backend = {half ? "cuda:half" : "cuda:float"};
  ctx.array_class = "CudaCachedArray";
  ctx.device_id = std::to_string(device);
  const vector<int> p(pad, pad + spatial_dims), s(stride, stride + spatial_dims), d(dilation, dilation + spatial_dims);
  if (half)
    return static_cast<Function *>(new FusedDwBnQuantCuda<Half>(
        ctx, base_axis, p, s, d, multiplier, with_bias != 0, bn_eps, no_scale != 0, no_bias != 0, quant_kind,
        sign != 0, with_zero != 0, n, m, delta, decay, x_min_max != 0, ema != 0, mm_eps));
  return static_cast<Function *>(new FusedDwBnQuantCuda<float>(
      ctx, base_axis, p, s, d, multiplier, with_bias != 0, bn_eps, no_scale != 0, no_bias != 0, quant_kind,
      sign != 0, with_zero != 0, n, m, delta, decay, x_min_max != 0, ema != 0, mm_eps));
}

// Factory of the pointwise function object (the converter that replaces a matched
// Convolution 1x1 -> BatchNormalization -> [ReLU | ReLU6] -> quantizer chain calls it). act is a
// dwbnq_act, quant_kind a dwbnq_quant_kind other than MINMAX; returns NULL on a bad argument.
extern "C" void *dwbnq_nbla_create_fused_pw(int half, int device, int base_axis, int with_bias, float bn_eps,
                                            int no_scale, int no_bias, int act, int quant_kind, int sign,
                                            int with_zero, int n, int m, float delta, int allow_tf32) {
  using namespace nbla;
  using namespace dwbnq_nbla;
  if (base_axis < 0 || device < 0 || act < DWBNQ_ACT_NONE || act > DWBNQ_ACT_RELU6 || quant_kind < DWBNQ_Q_NONE ||
      quant_kind > DWBNQ_Q_POW2)
    return nullptr;
  Context ctx;
  ctx.backend = {half ? "cuda:half" : "cuda:float"};
  ctx.array_class = "CudaCachedArray";
  ctx.device_id = std::to_string(device);
  if (half)
    return static_cast<Function *>(new FusedPwBnQuantCuda<Half>(ctx, base_axis, with_bias != 0, bn_eps, no_scale != 0,
                                                                no_bias != 0, act, quant_kind, sign != 0,
                                                                with_zero != 0, n, m, delta, allow_tf32 != 0));
  return static_cast<Function *>(new FusedPwBnQuantCuda<float>(ctx, base_axis, with_bias != 0, bn_eps, no_scale != 0,
                                                               no_bias != 0, act, quant_kind, sign != 0, with_zero != 0,
                                                               n, m, delta, allow_tf32 != 0));
}

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
