// TEST INFRASTRUCTURE: drives the dwbnq registry plugin through the stand-in nnabla interface
// of nbla/stub_core.hpp. Built by tests/test_nbla_plugin.py together with the plugin source;
// the functions are created through the (stub) registry under the reference's class names and
// run on caller-provided device buffers.
#include <cstring>
#include <nbla/stub_core.hpp>

extern "C" void dwbnq_register_nbla(void);
extern "C" void *dwbnq_nbla_create_fused_pw(int half, int device, int base_axis, int with_bias, float bn_eps, int no_scale,
                                            int no_bias, int act, int quant_kind, int sign, int with_zero, int n, int m,
                                            float delta, int allow_tf32);
extern "C" void *dwbnq_nbla_create_fused(int half, int device, int base_axis, int spatial_dims, const int *pad,
                                         const int *stride, const int *dilation, int multiplier, int with_bias,
                                         float bn_eps, int no_scale, int no_bias, int quant_kind, int sign,
                                         int with_zero, int n, int m, float delta, float decay, int x_min_max,
                                         int ema, float mm_eps);

namespace {
thread_local std::string g_err;
nbla::Context ctx_for(int device, int half) {
  nbla::Context c;
  c.backend = {half ? "cuda:half" : "cuda:float"};
  c.array_class = "CudaCachedArray";
  c.device_id = std::to_string(device);
  return c;
}
template <typename F> int guarded(F &&f) {
  try {
    f();
    return 0;
  } catch (const nbla::Exception &e) {
    g_err = e.what();
    return 100 + (int)e.code;
  } catch (const std::exception &e) {
    g_err = e.what();
    return 1;
  }
}
nbla::Shape_t shp(const int64_t *s, int n) { return nbla::Shape_t(s, s + n); }
}  // namespace

extern "C" {
const char *stub_last_error(void) { return g_err.c_str(); }
// scratch for Variables the functions allocate themselves (MinMaxQuantize's workspace)
void stub_set_scratch(void *p) {
  nbla::Variable::default_alloc() = [p](size_t) { return p; };
}
int stub_registered(const char *base, const char *backend) {
  dwbnq_register_nbla();
  return nbla::StubRegistry::table().count(std::string(base) + "/" + backend) ? 1 : 0;
}
int stub_name(const char *backend, int device, char *out, int cap) {
  return guarded([&] {
    dwbnq_register_nbla();
    std::unique_ptr<nbla::Function> f(nbla::stub_create<bool, int, float, bool>(
        "FixedPointQuantize", backend, ctx_for(device, 0), true, 8, 0.0625f, true));
    std::strncpy(out, f->name().c_str(), cap - 1);
    out[cap - 1] = 0;
  });
}
int stub_dwconv(int half, int device, const int64_t *xs, const int64_t *ws, int nd, void *x, void *w, void *b, void *y,
                int pad, int stride, int dil, int mult) {
  return guarded([&] {
    dwbnq_register_nbla();
    const std::vector<int> p(nd - 2, pad), s(nd - 2, stride), d(nd - 2, dil);
    std::unique_ptr<nbla::Function> f(
        nbla::stub_create<int, const std::vector<int> &, const std::vector<int> &, const std::vector<int> &, int>(
            "DepthwiseConvolution", half ? "cuda:half" : "cuda:float", ctx_for(device, half), 1, p, s, d, mult));
    nbla::Variable vx(shp(xs, nd), x), vw(shp(ws, nd - 1), w), vb(nbla::Shape_t{ws[0]}, b), vy(nbla::Shape_t{}, y);
    nbla::Variables in{&vx, &vw};
    if (b) in.push_back(&vb);
    nbla::Variables out{&vy};
    f->setup(in, out);
    f->forward(in, out);
  });
}
int stub_bn(int half, int device, const int64_t *xs, int nd, void *x, void *beta, void *gamma, void *mean, void *var,
            void *y, float eps, int batch_stat) {
  return guarded([&] {
    dwbnq_register_nbla();
    std::unique_ptr<nbla::Function> f(nbla::stub_create<const std::vector<int> &, float, float, bool, bool, bool>(
        "BatchNormalization", half ? "cuda:half" : "cuda:float", ctx_for(device, half), std::vector<int>{1}, 0.9f, eps,
        batch_stat != 0, gamma == nullptr, beta == nullptr));
    nbla::Shape_t ps(nd, 1);
    ps[1] = xs[1];
    nbla::Variable vx(shp(xs, nd), x), vb(ps, beta), vg(ps, gamma), vm(ps, mean), vv(ps, var), vy(shp(xs, nd), y);
    nbla::Variables in{&vx};
    if (beta) in.push_back(&vb);
    if (gamma) in.push_back(&vg);
    in.push_back(&vm);
    in.push_back(&vv);
    nbla::Variables out{&vy};
    f->setup(in, out);
    f->forward(in, out);
  });
}
int stub_fpq(int half, int device, int64_t size, void *x, void *y, int sign, int n, float delta) {
  return guarded([&] {
    dwbnq_register_nbla();
    std::unique_ptr<nbla::Function> f(nbla::stub_create<bool, int, float, bool>(
        "FixedPointQuantize", half ? "cuda:half" : "cuda:float", ctx_for(device, half), sign != 0, n, delta, true));
    nbla::Variable vx(nbla::Shape_t{size}, x), vy(nbla::Shape_t{size}, y);
    nbla::Variables in{&vx}, out{&vy};
    f->setup(in, out);
    f->forward(in, out);
  });
}
int stub_pow2(int half, int device, int64_t size, void *x, void *y, int sign, int with_zero, int n, int m) {
  return guarded([&] {
    dwbnq_register_nbla();
    std::unique_ptr<nbla::Function> f(nbla::stub_create<bool, bool, int, int, bool>(
        "Pow2Quantize", half ? "cuda:half" : "cuda:float", ctx_for(device, half), sign != 0, with_zero != 0, n, m, true));
    nbla::Variable vx(nbla::Shape_t{size}, x), vy(nbla::Shape_t{size}, y);
    nbla::Variables in{&vx}, out{&vy};
    f->setup(in, out);
    f->forward(in, out);
  });
}
int stub_minmax(int half, int device, const int64_t *xs, int nd, void *x, void *qr_min, void *qr_max, void *ql_min,
                void *ql_max, void *y, float decay, int x_min_max, int ema, float eps) {
  return guarded([&] {
    dwbnq_register_nbla();
    std::unique_ptr<nbla::Function> f(nbla::stub_create<float, bool, bool, bool, float>(
        "MinMaxQuantize", half ? "cuda:half" : "cuda:float", ctx_for(device, half), decay, x_min_max != 0, ema != 0, true, eps));
    nbla::Shape_t ps(nd, 1);
    ps[1] = xs[1];
    nbla::Variable vx(shp(xs, nd), x), a(ps, qr_min), b(ps, qr_max), c(ps, ql_min), d(ps, ql_max), vy(shp(xs, nd), y);
    nbla::Variables in{&vx, &a, &b, &c, &d}, out{&vy};
    f->setup(in, out);
    f->forward(in, out);
  });
}
// The fused function object through its factory: inputs in the order of the three functions
// it replaces; ptrs = {x, w, b, beta, gamma, mean, var, qr_min, qr_max, ql_min, ql_max} with
// null for an absent optional input. The output Variable starts without a shape: setup
// must derive it (out_shape receives it).
int stub_fused(int half, int device, const int64_t *xs, const int64_t *ws, int nd, void *const *ptrs, void *y,
               int pad, int stride, float bn_eps, int quant_kind, int sign, int with_zero, int n, int m, float delta,
               float decay, int x_min_max, int ema, float mm_eps, int64_t *out_shape, int *n_inputs, int *copies_ok) {
  return guarded([&] {
    const int p[2] = {pad, pad}, s[2] = {stride, stride}, d[2] = {1, 1};
    nbla::Function *raw = static_cast<nbla::Function *>(dwbnq_nbla_create_fused(
        half, device, 1, nd - 2, p, s, d, 1, ptrs[2] != nullptr, bn_eps, ptrs[4] == nullptr, ptrs[3] == nullptr,
        quant_kind, sign, with_zero, n, m, delta, decay, x_min_max, ema, mm_eps));
    if (!raw) throw std::runtime_error("factory returned null");
    std::unique_ptr<nbla::Function> f(raw);
    nbla::Shape_t ps(nd, 1);
    ps[1] = ws[0];
    nbla::Variable vx(shp(xs, nd), ptrs[0]), vw(shp(ws, nd - 1), ptrs[1]), vb(nbla::Shape_t{ws[0]}, ptrs[2]);
    nbla::Variable vbeta(ps, ptrs[3]), vgamma(ps, ptrs[4]), vmean(ps, ptrs[5]), vvar(ps, ptrs[6]);
    nbla::Variable r0(ps, ptrs[7]), r1(ps, ptrs[8]), r2(ps, ptrs[9]), r3(ps, ptrs[10]);
    nbla::Variable vy(nbla::Shape_t{}, y);
    nbla::Variables in{&vx, &vw};
    if (ptrs[2]) in.push_back(&vb);
    if (ptrs[3]) in.push_back(&vbeta);
    if (ptrs[4]) in.push_back(&vgamma);
    in.push_back(&vmean);
    in.push_back(&vvar);
    if (quant_kind == 3) {
      in.push_back(&r0);
      in.push_back(&r1);
      in.push_back(&r2);
      in.push_back(&r3);
    }
    *n_inputs = f->min_inputs();
    nbla::Variables out{&vy};
    // a copy (what nnabla makes when a graph is cloned) must behave like the original
    std::shared_ptr<nbla::Function> g = f->copy();
    *copies_ok = g && g->name() == f->name() && g->min_inputs() == f->min_inputs() &&
                 g->in_types().size() == (size_t)f->min_inputs() && g->out_types().size() == 1;
    g->setup(in, out);
    g->forward(in, out);
    const nbla::Shape_t ys = vy.shape();
    for (int i = 0; i < nd; ++i) out_shape[i] = i < (int)ys.size() ? ys[i] : -1;
  });
}
// The pointwise function object: ptrs = {x, w, b, beta, gamma, mean, var}, null for an absent
// optional input; ws is [c_out, c_in, 1, 1].
int stub_fused_pw(int half, int device, const int64_t *xs, const int64_t *ws, void *const *ptrs, void *y, float bn_eps,
                  int act, int quant_kind, int sign, int with_zero, int n, int m, float delta, int allow_tf32,
                  int64_t *out_shape, int *n_inputs, int *copies_ok) {
  return guarded([&] {
    nbla::Function *raw = static_cast<nbla::Function *>(
        dwbnq_nbla_create_fused_pw(half, device, 1, ptrs[2] != nullptr, bn_eps, ptrs[4] == nullptr, ptrs[3] == nullptr, act,
                                   quant_kind, sign, with_zero, n, m, delta, allow_tf32));
    if (!raw) throw std::runtime_error("factory returned null");
    std::unique_ptr<nbla::Function> f(raw);
    nbla::Shape_t ps(4, 1);
    ps[1] = ws[0];
    nbla::Variable vx(shp(xs, 4), ptrs[0]), vw(shp(ws, 4), ptrs[1]), vb(nbla::Shape_t{ws[0]}, ptrs[2]);
    nbla::Variable vbeta(ps, ptrs[3]), vgamma(ps, ptrs[4]), vmean(ps, ptrs[5]), vvar(ps, ptrs[6]);
    nbla::Variable vy(nbla::Shape_t{}, y);
    nbla::Variables in{&vx, &vw};
    if (ptrs[2]) in.push_back(&vb);
    if (ptrs[3]) in.push_back(&vbeta);
    if (ptrs[4]) in.push_back(&vgamma);
    in.push_back(&vmean);
    in.push_back(&vvar);
    *n_inputs = f->min_inputs();
    nbla::Variables out{&vy};
    std::shared_ptr<nbla::Function> g = f->copy();
    *copies_ok = g && g->name() == f->name() && g->min_inputs() == f->min_inputs() &&
                 g->in_types().size() == (size_t)f->min_inputs() && g->out_types().size() == 1;
    g->setup(in, out);
    g->forward(in, out);
    const nbla::Shape_t ys = vy.shape();
    for (int i = 0; i < 4; ++i) out_shape[i] = i < (int)ys.size() ? ys[i] : -1;
  });
}
int stub_fused_backward_is_refused(int device) {
  return guarded([&] {
    const int p[2] = {1, 1}, s[2] = {1, 1}, d[2] = {1, 1};
    std::unique_ptr<nbla::Function> f(static_cast<nbla::Function *>(dwbnq_nbla_create_fused(
        0, device, 1, 2, p, s, d, 1, 1, 1e-5f, 0, 0, 1, 1, 0, 8, 0, 0.0625f, 0.f, 0, 0, 0.f)));
    f->backward({}, {}, {}, {});
  });
}
int stub_backward_is_refused(int device) {
  return guarded([&] {
    dwbnq_register_nbla();
    std::unique_ptr<nbla::Function> f(nbla::stub_create<float, bool, bool, bool, float>(
        "MinMaxQuantize", "cuda:float", ctx_for(device, 0), 0.999f, true, false, true, 0.01f));
    f->backward({}, {}, {}, {});
  });
}
// backward of the two quantizers through the registered classes: which = 0 FixedPointQuantize
// (sign, n, delta), 1 Pow2Quantize (sign, with_zero = a, n, m = b)
int stub_quant_bwd(int which, int half, int device, int64_t size, void *x, void *dy, void *dx, int sign, int n, float delta,
                   int a, int b, int fine, int accum, int propagate) {
  return guarded([&] {
    dwbnq_register_nbla();
    const char *be = half ? "cuda:half" : "cuda:float";
    std::unique_ptr<nbla::Function> f(
        which == 0 ? nbla::stub_create<bool, int, float, bool>("FixedPointQuantize", be, ctx_for(device, half), sign != 0, n,
                                                               delta, fine != 0)
                   : nbla::stub_create<bool, bool, int, int, bool>("Pow2Quantize", be, ctx_for(device, half), sign != 0,
                                                                   a != 0, n, b, fine != 0));
    nbla::Variable vx(nbla::Shape_t{size}, x), vy(nbla::Shape_t{size}, nullptr);
    vx.set_grad(dx);
    vy.set_grad(dy);
    nbla::Variables in{&vx}, out{&vy};
    f->setup(in, out);
    f->backward(in, out, {propagate != 0}, {accum != 0});
  });
}
int stub_dwconv_bwd(int half, int device, const int64_t *xs, const int64_t *ws, int nd, void *x, void *w, void *b, void *dy,
                    void *dx, void *dw, void *db, int pad, int stride, int dil, int mult, int propagate_mask,
                    int accum_mask) {
  return guarded([&] {
    dwbnq_register_nbla();
    const std::vector<int> p(nd - 2, pad), s(nd - 2, stride), d(nd - 2, dil);
    std::unique_ptr<nbla::Function> f(
        nbla::stub_create<int, const std::vector<int> &, const std::vector<int> &, const std::vector<int> &, int>(
            "DepthwiseConvolution", half ? "cuda:half" : "cuda:float", ctx_for(device, half), 1, p, s, d, mult));
    nbla::Variable vx(shp(xs, nd), x), vw(shp(ws, nd - 1), w), vb(nbla::Shape_t{ws[0]}, b), vy(nbla::Shape_t{}, nullptr);
    vx.set_grad(dx);
    vw.set_grad(dw);
    vb.set_grad(db);
    vy.set_grad(dy);
    nbla::Variables in{&vx, &vw};
    if (b) in.push_back(&vb);
    nbla::Variables out{&vy};
    f->setup(in, out);
    std::vector<bool> pd, ac;
    for (size_t i = 0; i < in.size(); ++i) {
      pd.push_back((propagate_mask >> i) & 1);
      ac.push_back((accum_mask >> i) & 1);
    }
    f->backward(in, out, pd, ac);
  });
}
}
