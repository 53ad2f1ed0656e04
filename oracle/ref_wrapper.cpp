// TEST INFRASTRUCTURE — not part of the product.
//
// C-ABI wrapper around the *reference's own* CPU implementation of the convolution hot path, compiled in
// place from the reference source tree (see oracle/build.py).  It instantiates the reference classes
// unmodified:
//   ParallelizedBridge<float, ConvolutionBridge>  (src/bridges/ParallelizedBridge.h:303-320)
//   ConvolutionBridge<..., CPUDriver>             (src/bridges/ConvolutionBridge_impl.hxx:294-373, 551-628)
//   MaxPoolingBridge / ReLUBridge                 (src/bridges/MaxPoolingBridge_impl.hxx, ReLUBridge_impl.hxx)
//   LRNBridge / DropoutBridge / FullyConnectedBridge / SoftmaxLossBridge   (src/bridges/*_impl.hxx)
// and copies caller buffers in and out of the reference's cubes.  Only tests, the smoke check and the
// CPU-baseline leg of the benchmark may load the resulting library.
#include <chrono>
#include <cstring>
#include <iostream>
#include <thread>
#include <vector>

#include "bridges/ParallelizedBridge.h"
#include "bridges/ConvolutionBridge.h"
#include "bridges/MaxPoolingBridge.h"
#include "bridges/ReLUBridge.h"
#include "bridges/LRNBridge.h"
#include "bridges/DropoutBridge.h"
#include "bridges/FullyConnectedBridge.h"
#include "bridges/SoftmaxLossBridge.h"

namespace {

typedef LogicalCube<float, Layout_CRDB> Cube;
typedef Layer<float, Layout_CRDB> CubeLayer;
typedef ParallelizedBridge<float, ConvolutionBridge> PConv;

struct ConvHandle {
  int B, D, n, o, k, s, p, m;
  Cube *x, *dx, *y, *dy;
  CubeLayer *lin, *lout;
  cnn::LayerParameter lp;
  cnn::SolverParameter sp;
  CPUDriver drv;
  PConv* bridge;
};

// The pooling bridge keeps its arg-max cube protected; a derived type reads it (declared size_t, used as int32:
// src/bridges/MaxPoolingBridge.h:92, MaxPoolingBridge_impl.hxx:79-81).
struct PoolWithIndex : MaxPoolingBridge<float, Layout_CRDB, float, Layout_CRDB, CPUDriver> {
  using MaxPoolingBridge<float, Layout_CRDB, float, Layout_CRDB, CPUDriver>::MaxPoolingBridge;
  const int* indices() const { return (const int*)this->max_index->get_p_data(); }
};

double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// Runs fwd (+ bwd when `with_backward`) of a bridge once for the results, then `iters` more times for the clock;
// returns the median seconds of one fwd+bwd pair (0 when iters == 0).
template <class Bridge>
static double run_and_time(Bridge& br, bool with_backward, int iters, void (*after_first)(void*), void* arg) {
  br.forward();
  if (with_backward) br.backward();
  if (after_first) after_first(arg);
  std::vector<double> tt;
  for (int i = 0; i < iters; ++i) {
    const double t0 = now_s();
    br.forward();
    if (with_backward) br.backward();
    tt.push_back(now_s() - t0);
  }
  if (tt.empty()) return 0.0;
  std::sort(tt.begin(), tt.end());
  return tt[tt.size() / 2];
}

}  // namespace

extern "C" {

int cctref_hardware_concurrency() { return (int)std::thread::hardware_concurrency(); }

const char* cctref_blas_config() { return openblas_get_config(); }

// Largest power of two <= hardware_concurrency, capped by the batch: the partition count DeepNet uses for
// convolution layers (src/DeepNet.h:716-725, 1102-1105).
int cctref_default_partitions(int batch) {
  unsigned hc = std::thread::hardware_concurrency();
  int p = 1;
  while ((unsigned)(p * 2) <= hc) p *= 2;
  return p < batch ? p : batch;
}

void* cctref_conv_create(int B, int D, int n, int o, int k, int s, int p, int bias_term, int n_partition,
                         int needs_dx, float base_lr, float momentum, float weight_decay) {
  ConvHandle* h = new ConvHandle();
  h->B = B; h->D = D; h->n = n; h->o = o; h->k = k; h->s = s; h->p = p;
  h->m = (n + 2 * p - k) / s + 1;
  h->x = new Cube(n, n, D, B);
  h->dx = new Cube(n, n, D, B);
  h->y = new Cube(h->m, h->m, o, B);
  h->dy = new Cube(h->m, h->m, o, B);
  h->lin = new CubeLayer(h->x, h->dx);
  h->lout = new CubeLayer(h->y, h->dy);
  h->lp.conv_.num_output_ = o;
  h->lp.conv_.kernel_size_ = k;
  h->lp.conv_.stride_ = s;
  h->lp.conv_.pad_ = p;
  h->lp.conv_.bias_term_ = bias_term != 0;
  h->sp.base_lr_ = base_lr;
  h->sp.momentum_ = momentum;
  h->sp.weight_decay_ = weight_decay;
  h->sp.lr_policy_ = "step";
  h->sp.gamma_ = 0.1f;
  h->sp.stepsize_ = 100000;
  h->sp.random_seed_ = 1;
  std::streambuf* keep = std::cout.rdbuf(nullptr);  // the bridge constructors narrate on stdout
  h->bridge = new PConv(h->lin, h->lout, &h->lp, &h->sp, &h->drv, (size_t)n_partition, 1);
  std::cout.rdbuf(keep);
  std::cout.clear();
  h->bridge->needs_to_calc_backward_grad = needs_dx != 0;
  return h;
}

void cctref_conv_destroy(void* hv) {
  ConvHandle* h = (ConvHandle*)hv;
  delete h->bridge;
  delete h->lin; delete h->lout;  // a Layer deletes its two cubes (src/Layer.h:57-59)
  delete h;
}

void cctref_conv_set_model(void* hv, const float* W, const float* bias) {
  ConvHandle* h = (ConvHandle*)hv;
  std::memcpy(h->bridge->get_model_cube()->get_p_data(), W, sizeof(float) * h->o * h->D * h->k * h->k);
  if (bias && h->bridge->get_bias_cube())
    std::memcpy(h->bridge->get_bias_cube()->get_p_data(), bias, sizeof(float) * h->o);
}

void cctref_conv_get_model(void* hv, float* W, float* bias) {
  ConvHandle* h = (ConvHandle*)hv;
  std::memcpy(W, h->bridge->get_model_cube()->get_p_data(), sizeof(float) * h->o * h->D * h->k * h->k);
  if (bias && h->bridge->get_bias_cube())
    std::memcpy(bias, h->bridge->get_bias_cube()->get_p_data(), sizeof(float) * h->o);
}

void cctref_conv_forward(void* hv, const float* X, float* Y) {
  ConvHandle* h = (ConvHandle*)hv;
  std::memcpy(h->x->get_p_data(), X, sizeof(float) * h->x->n_elements);
  h->bridge->forward();
  std::memcpy(Y, h->y->get_p_data(), sizeof(float) * h->y->n_elements);
}

// forward() must have been called on the same X before (the CPU bridge keeps the lowered input).
// do_update != 0 lets the reference apply its SGD step to the model held by the bridge.
void cctref_conv_backward(void* hv, const float* dY, float* dX, float* dW, float* db, int do_update) {
  ConvHandle* h = (ConvHandle*)hv;
  std::memcpy(h->dy->get_p_data(), dY, sizeof(float) * h->dy->n_elements);
  h->bridge->set_update_model_gradients(do_update != 0);
  h->bridge->backward();
  if (dX) std::memcpy(dX, h->dx->get_p_data(), sizeof(float) * h->dx->n_elements);
  if (dW) std::memcpy(dW, h->bridge->get_model_gradient_host(), sizeof(float) * h->o * h->D * h->k * h->k);
  if (db && h->bridge->get_bias_cube()) std::memcpy(db, h->bridge->get_bias_gradient_host(), sizeof(float) * h->o);
}

// Times forward()+backward() on whatever the cubes currently hold (no copies inside the timed region, no SGD).
// Returns the median seconds of `iters` fwd+bwd pairs after `warmup` untimed ones; per-pass medians via out-params.
double cctref_conv_time(void* hv, int warmup, int iters, double* fwd_s, double* bwd_s) {
  ConvHandle* h = (ConvHandle*)hv;
  h->bridge->set_update_model_gradients(false);
  std::vector<double> tf, tb, tt;
  for (int i = 0; i < warmup + iters; ++i) {
    double t0 = now_s();
    h->bridge->forward();
    double t1 = now_s();
    h->bridge->backward();
    double t2 = now_s();
    if (i >= warmup) { tf.push_back(t1 - t0); tb.push_back(t2 - t1); tt.push_back(t2 - t0); }
  }
  std::sort(tf.begin(), tf.end()); std::sort(tb.begin(), tb.end()); std::sort(tt.begin(), tt.end());
  if (fwd_s) *fwd_s = tf[tf.size() / 2];
  if (bwd_s) *bwd_s = tb[tb.size() / 2];
  return tt[tt.size() / 2];
}

// One training step on whatever the cubes hold: forward, backward and (do_update != 0) the reference's SGD update.
void cctref_conv_step(void* hv, int do_update) {
  ConvHandle* h = (ConvHandle*)hv;
  h->bridge->set_update_model_gradients(do_update != 0);
  h->bridge->forward();
  h->bridge->backward();
}

// Fill the bridge's cubes for timing without going through forward()/backward() copies.
void cctref_conv_load(void* hv, const float* X, const float* dY) {
  ConvHandle* h = (ConvHandle*)hv;
  if (X) std::memcpy(h->x->get_p_data(), X, sizeof(float) * h->x->n_elements);
  if (dY) std::memcpy(h->dy->get_p_data(), dY, sizeof(float) * h->dy->n_elements);
}

// Max pooling through the reference bridge: Y and idx (int32 offset inside each n x n plane) from X,
// then dX from dY.  Pass dY == NULL to skip the backward half.
void cctref_maxpool(int B, int D, int n, int k, int s, const float* X, float* Y, int* idx, const float* dY,
                    float* dX) {
  int m = (n - k) / s + 1;
  Cube &x = *new Cube(n, n, D, B), &dx = *new Cube(n, n, D, B), &y = *new Cube(m, m, D, B), &dy = *new Cube(m, m, D, B);
  CubeLayer lin(&x, &dx), lout(&y, &dy);  // the Layers delete the cubes
  cnn::LayerParameter lp;
  lp.pool_.kernel_size_ = k;
  lp.pool_.stride_ = s;
  cnn::SolverParameter sp;
  CPUDriver drv;
  PoolWithIndex br(&lin, &lout, &lp, &sp, &drv);
  std::memcpy(x.get_p_data(), X, sizeof(float) * x.n_elements);
  br.forward();
  std::memcpy(Y, y.get_p_data(), sizeof(float) * y.n_elements);
  if (idx) std::memcpy(idx, br.indices(), sizeof(int) * y.n_elements);
  if (dY && dX) {
    std::memcpy(dy.get_p_data(), dY, sizeof(float) * dy.n_elements);
    br.backward();
    std::memcpy(dX, dx.get_p_data(), sizeof(float) * dx.n_elements);
  }
}

// ReLU through the reference bridge: Y = max(X, 0); dX = dY * [X > 0] (pass dY == NULL to skip).
void cctref_relu(int B, int D, int n, const float* X, float* Y, const float* dY, float* dX) {
  Cube &x = *new Cube(n, n, D, B), &dx = *new Cube(n, n, D, B), &y = *new Cube(n, n, D, B), &dy = *new Cube(n, n, D, B);
  CubeLayer lin(&x, &dx), lout(&y, &dy);  // the Layers delete the cubes
  cnn::LayerParameter lp;
  cnn::SolverParameter sp;
  CPUDriver drv;
  ReLUBridge<float, Layout_CRDB, float, Layout_CRDB, CPUDriver> br(&lin, &lout, &lp, &sp, &drv);
  std::memcpy(x.get_p_data(), X, sizeof(float) * x.n_elements);
  br.forward();
  std::memcpy(Y, y.get_p_data(), sizeof(float) * y.n_elements);
  if (dY && dX) {
    std::memcpy(dy.get_p_data(), dY, sizeof(float) * dy.n_elements);
    br.backward();
    std::memcpy(dX, dx.get_p_data(), sizeof(float) * dx.n_elements);
  }
}

// Across-channel LRN through the reference bridge: Y from X, then dX from dY (pass dY == NULL to skip).
double cctref_lrn(int B, int D, int n, int local_size, float alpha, float beta, const float* X, float* Y,
                  const float* dY, float* dX, int time_iters) {
  Cube &x = *new Cube(n, n, D, B), &dx = *new Cube(n, n, D, B), &y = *new Cube(n, n, D, B), &dy = *new Cube(n, n, D, B);
  CubeLayer lin(&x, &dx), lout(&y, &dy);
  cnn::LayerParameter lp;
  lp.lrn_.local_size_ = local_size; lp.lrn_.alpha_ = alpha; lp.lrn_.beta_ = beta;
  cnn::SolverParameter sp;
  CPUDriver drv;
  LRNBridge<float, Layout_CRDB, float, Layout_CRDB, CPUDriver> br(&lin, &lout, &lp, &sp, &drv);
  std::memcpy(x.get_p_data(), X, sizeof(float) * x.n_elements);
  if (dY) std::memcpy(dy.get_p_data(), dY, sizeof(float) * dy.n_elements);
  br.forward();
  std::memcpy(Y, y.get_p_data(), sizeof(float) * y.n_elements);
  if (dY && dX) {
    br.backward();
    std::memcpy(dX, dx.get_p_data(), sizeof(float) * dx.n_elements);
  }
  return time_iters > 0 ? run_and_time(br, dY != NULL, time_iters, NULL, NULL) : 0.0;
}

// Dropout (training phase) through the reference bridge: the bridge draws its own mask from mt19937(seed); the mask
// it used is returned so that the same one can be given to the implementation under test.
double cctref_dropout(int B, int D, int n, float ratio, int seed, const float* X, float* Y, unsigned int* mask,
                      const float* dY, float* dX, int time_iters) {
  Cube &x = *new Cube(n, n, D, B), &dx = *new Cube(n, n, D, B), &y = *new Cube(n, n, D, B), &dy = *new Cube(n, n, D, B);
  CubeLayer lin(&x, &dx), lout(&y, &dy);
  cnn::LayerParameter lp;
  lp.dropout_.ratio_ = ratio;
  cnn::SolverParameter sp;
  sp.random_seed_ = seed;
  CPUDriver drv;
  DropoutBridge<float, Layout_CRDB, float, Layout_CRDB, CPUDriver> br(&lin, &lout, &lp, &sp, &drv);
  std::memcpy(x.get_p_data(), X, sizeof(float) * x.n_elements);
  br.forward();
  std::memcpy(Y, y.get_p_data(), sizeof(float) * y.n_elements);
  if (mask) std::memcpy(mask, br.mask_cube->get_p_data(), sizeof(unsigned int) * x.n_elements);
  if (dY && dX) {
    std::memcpy(dy.get_p_data(), dY, sizeof(float) * dy.n_elements);
    br.backward();
    std::memcpy(dX, dx.get_p_data(), sizeof(float) * dx.n_elements);
  }
  return time_iters > 0 ? run_and_time(br, dY != NULL, time_iters, NULL, NULL) : 0.0;
}

// Fully connected layer through the reference bridge (no SGD step: the bare bridge has no updater).
double cctref_fc(int B, int D, int n, int o, const float* X, const float* W, const float* bias, float* Y, const float* dY,
                 float* dX, float* dW, float* db, int blas_threads, int time_iters) {
  Cube &x = *new Cube(n, n, D, B), &dx = *new Cube(n, n, D, B), &y = *new Cube(1, 1, o, B), &dy = *new Cube(1, 1, o, B);
  CubeLayer lin(&x, &dx), lout(&y, &dy);
  cnn::LayerParameter lp;
  lp.ip_.num_output_ = o;
  lp.ip_.bias_term_ = bias != NULL;
  cnn::SolverParameter sp;
  sp.random_seed_ = 1;
  CPUDriver drv;
  std::streambuf* keep = std::cout.rdbuf(nullptr);
  FullyConnectedBridge<float, Layout_CRDB, float, Layout_CRDB, CPUDriver> br(&lin, &lout, &lp, &sp, &drv);
  std::cout.rdbuf(keep);
  std::cout.clear();
  br.run_with_n_threads = blas_threads > 0 ? blas_threads : 1;
  std::memcpy(br.get_model_cube()->get_p_data(), W, sizeof(float) * (size_t)o * D * n * n);
  if (bias) std::memcpy(br.get_bias_cube()->get_p_data(), bias, sizeof(float) * o);
  std::memcpy(x.get_p_data(), X, sizeof(float) * x.n_elements);
  br.forward();
  if (Y) std::memcpy(Y, y.get_p_data(), sizeof(float) * y.n_elements);
  if (dY) {
    std::memcpy(dy.get_p_data(), dY, sizeof(float) * dy.n_elements);
    br.backward();
    if (dX) std::memcpy(dX, dx.get_p_data(), sizeof(float) * dx.n_elements);
    if (dW) std::memcpy(dW, br.get_model_grad_cube()->get_p_data(), sizeof(float) * (size_t)o * D * n * n);
    if (db && bias) std::memcpy(db, br.get_bias_grad_cube()->get_p_data(), sizeof(float) * o);
  }
  return time_iters > 0 ? run_and_time(br, dY != NULL, time_iters, NULL, NULL) : 0.0;
}

// Softmax with loss through the reference bridge: prob (the bridge's output cube), the summed loss, and the gradient
// with respect to the input (scaled by 1 / B as the bridge does).
double cctref_softmax_loss(int B, int C, const float* X, const float* labels, float* prob, float* loss, float* dX,
                           int time_iters) {
  Cube &x = *new Cube(1, 1, C, B), &dx = *new Cube(1, 1, C, B), &y = *new Cube(1, 1, C, B), &dy = *new Cube(1, 1, C, B);
  CubeLayer lin(&x, &dx), lout(&y, &dy);
  Cube lab(1, 1, 1, B);
  CPUDriver drv;
  SoftmaxLossBridge<float, Layout_CRDB, float, Layout_CRDB, CPUDriver> br(&lin, &lout, &lab, &drv);
  std::memcpy(x.get_p_data(), X, sizeof(float) * x.n_elements);
  std::memcpy(lab.get_p_data(), labels, sizeof(float) * B);
  br.forward();
  if (prob) std::memcpy(prob, y.get_p_data(), sizeof(float) * y.n_elements);
  if (loss) *loss = br.get_loss();
  if (dX) {
    br.backward();
    std::memcpy(dX, dx.get_p_data(), sizeof(float) * dx.n_elements);
  }
  return time_iters > 0 ? run_and_time(br, dX != NULL, time_iters, NULL, NULL) : 0.0;
}

// The reference's parameter fillers (CPUDriver::sgaussian_initialize / sinitialize_xavier / sbernoulli_initialize,
// src/sched/DeviceDriver_CPU.cpp:661-699) on a host buffer.  kind: 0 gaussian(a = mean, b = std), 1 xavier over
// n_batch filters, 2 bernoulli(a = p).
void cctref_fill(int kind, float* out, long n, float a, float b, int seed, long n_batch) {
  CPUDriver drv;
  DeviceMemoryPointer_Local_RAM ptr(out, sizeof(float) * (size_t)n);
  if (kind == 0) drv.sgaussian_initialize(&ptr, a, b, seed);
  else if (kind == 1) drv.sinitialize_xavier(&ptr, (size_t)n_batch, seed);
  else drv.sbernoulli_initialize(&ptr, a, seed);
}

}  // extern "C"

