// C++ host-side mirror of the reference types the convolution hot path touches, on top of the C ABI alone
// (include/cct_b200.h).  Member names and call order follow the reference so code written against it reads the same:
//   LogicalCube<T>            src/LogicalCube.h (R x C x D x B, "c" fastest = NCHW; owns memory iff built from sizes)
//   Layer                     src/Layer.h:36-37 (a data cube and a gradient cube)
//   PhysicalOperator          src/bridges/PhysicalOperator.h:15-30 (forward()/backward())
//   B200Driver                the slice of src/sched/DeviceDriver.h:56-274 the path needs
//   ConvolutionBridge         src/bridges/ConvolutionBridge.h + AbstractBridge.h members (iR..oB, p_*_layer,
//                             needs_to_calc_backward_grad, bias_term, model / bias / gradient cube accessors)
//   FullyConnectedBridge      src/bridges/FullyConnectedBridge.h, over the convolution plan (kernel = whole input)
//   SGDGradientUpdater        src/algorithms/GradientUpdater.h:154-193
//   Communicator              the C ABI's NCCL communicator (cct_comm_*): one per driver / GPU
//   ParallelizedBridge        one partition per GPU (one per process, or one per host thread as the reference's
//                             PhysicalStratum runs them): owns model, gradient and history, sums gradients over the
//                             partitions with an NCCL all-reduce (in place of src/bridges/ParallelizedBridge_impl.hxx:876-971:
//                             device-to-host gather + serial CPU sum), then updates on the device
// Errors: the reference's convention is print + assert(false) (src/sched/DeviceDriver.h:48-51); here the failing call
// prints the library's message and aborts, unless a handler was installed with B200Driver::set_error_handler.
#pragma once
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "../../include/cct_b200.h"

namespace cct {

class B200Driver {
 public:
  typedef void (*ErrorHandler)(int code, const char* what, const char* detail);
  explicit B200Driver(int device = 0, void* cuda_stream = nullptr, bool own_stream = true) {
    const int rc = own_stream ? cct_ctx_create(device, &ctx_) : cct_ctx_create_on_stream(device, cuda_stream, &ctx_);
    if (rc != CCT_OK) fail(rc, "cct_ctx_create");
  }
  ~B200Driver() {
    if (ctx_) cct_ctx_destroy(ctx_);
  }
  B200Driver(const B200Driver&) = delete;
  B200Driver& operator=(const B200Driver&) = delete;

  void* malloc(size_t bytes) { void* p = nullptr; check(cct_malloc(ctx_, bytes, &p), "cct_malloc"); return p; }
  void free(void* p) { check(cct_free(ctx_, p), "cct_free"); }
  void memcpy_h2d(void* dst, const void* src, size_t bytes) { check(cct_memcpy_h2d(ctx_, dst, src, bytes), "cct_memcpy_h2d"); }
  void memcpy_d2h(void* dst, const void* src, size_t bytes) { check(cct_memcpy_d2h(ctx_, dst, src, bytes), "cct_memcpy_d2h"); }
  void memset(void* p, int v, size_t bytes) { check(cct_memset(ctx_, p, v, bytes), "cct_memset"); }
  void sconstant_initialize(float* p, size_t count, float v) { check(cct_fill_f32(ctx_, p, count, v), "cct_fill_f32"); }
  void device_sync() { check(cct_sync(ctx_), "cct_sync"); }
  cct_ctx* ctx() const { return ctx_; }

  void check(int rc, const char* what) {
    if (rc != CCT_OK) fail(rc, what);
  }
  static void set_error_handler(ErrorHandler h) { handler() = h; }

 private:
  static ErrorHandler& handler() { static ErrorHandler h = nullptr; return h; }
  void fail(int rc, const char* what) {
    const char* detail = ctx_ ? cct_last_error_string(ctx_) : "";
    if (handler()) { handler()(rc, what, detail); return; }
    std::fprintf(stderr, "cct_b200: %s failed with code %d: %s\n", what, rc, detail);
    std::abort();
  }
  cct_ctx* ctx_ = nullptr;
};

template <typename T>
class LogicalCube {
 public:
  const size_t R, C, D, B, n_elements;
  LogicalCube(size_t r, size_t c, size_t d, size_t b, B200Driver* driver)
      : R(r), C(c), D(d), B(b), n_elements(r * c * d * b), p_driver_(driver), own_data_(true) {
    p_data_ = static_cast<T*>(driver->malloc(n_elements * sizeof(T)));
  }
  LogicalCube(T* data, size_t r, size_t c, size_t d, size_t b, B200Driver* driver)
      : R(r), C(c), D(d), B(b), n_elements(r * c * d * b), p_driver_(driver), own_data_(false), p_data_(data) {}
  ~LogicalCube() {
    if (own_data_ && p_data_) p_driver_->free(p_data_);
  }
  LogicalCube(const LogicalCube&) = delete;
  T* get_p_data() const { return p_data_; }
  void set_p_data(T* data) {  // an owning cube releases its memory first (src/LogicalCube_impl.hxx:20-34)
    if (own_data_ && p_data_) p_driver_->free(p_data_);
    own_data_ = false;
    p_data_ = data;
  }
  void reset_cube(T v = T(0)) { p_driver_->sconstant_initialize(reinterpret_cast<float*>(p_data_), n_elements, (float)v); }
  void copy_from_host(const T* src) { p_driver_->memcpy_h2d(p_data_, src, n_elements * sizeof(T)); p_driver_->device_sync(); }
  void copy_to_host(T* dst) const { p_driver_->memcpy_d2h(dst, p_data_, n_elements * sizeof(T)); p_driver_->device_sync(); }

 private:
  B200Driver* p_driver_;
  bool own_data_;
  T* p_data_ = nullptr;
};

struct Layer {
  LogicalCube<float>* const p_data_cube;
  LogicalCube<float>* const p_gradient_cube;
  Layer(LogicalCube<float>* data, LogicalCube<float>* grad) : p_data_cube(data), p_gradient_cube(grad) {}
};

class PhysicalOperator {
 public:
  int run_with_n_threads = 1;
  virtual void forward() = 0;
  virtual void backward() = 0;
  virtual ~PhysicalOperator() {}
};

// The convolution_param fields the bridge reads (src/bridges/ConvolutionBridge_impl.hxx:33-60).
struct ConvolutionParameter {
  int num_output = 0, kernel_size = 0, stride = 1, pad = 0, group = 1;
  bool bias_term = true;
};

class ConvolutionBridge : public PhysicalOperator {
 public:
  const size_t iR, iC, iD, iB, oR, oC, oD, oB;
  Layer* const p_input_layer;
  Layer* const p_output_layer;
  B200Driver* const p_driver;
  bool needs_to_calc_backward_grad = true;
  const bool bias_term;
  bool fuse_relu = false;  // fold the ReLU bridge that follows into the epilogue
  const size_t K, stride, padding, group;

  ConvolutionBridge(Layer* in, Layer* out, const ConvolutionParameter& cp, B200Driver* driver, int algo = CCT_ALGO_AUTO)
      : iR(in->p_data_cube->R), iC(in->p_data_cube->C), iD(in->p_data_cube->D), iB(in->p_data_cube->B),
        oR(out->p_data_cube->R), oC(out->p_data_cube->C), oD(out->p_data_cube->D), oB(out->p_data_cube->B),
        p_input_layer(in), p_output_layer(out), p_driver(driver), bias_term(cp.bias_term), K(cp.kernel_size),
        stride(cp.stride), padding(cp.pad), group(cp.group) {
    cct_conv_desc d = {(int)iB, (int)iD, (int)iR, (int)oD, cp.kernel_size, cp.stride, cp.pad, cp.group, cp.bias_term ? 1 : 0,
                       algo};
    int m = 0;
    driver->check(cct_conv_out_size(&d, &m), "cct_conv_out_size");
    if (iR != iC || (size_t)m != oR || oR != oC || iB != oB || (int)oD != cp.num_output)
      driver->check(CCT_ERR_INVALID, "ConvolutionBridge: layer shapes do not match the convolution");
    driver->check(cct_conv_plan_create(driver->ctx(), &d, &plan_), "cct_conv_plan_create");
    const size_t dg = iD / cp.group;
    p_model_cube_ = new LogicalCube<float>(K, K, dg, oD, driver);
    p_model_gradient_cube_ = new LogicalCube<float>(K, K, dg, oD, driver);
    if (bias_term) {
      p_bias_cube_ = new LogicalCube<float>(1, 1, oD, 1, driver);
      p_bias_gradient_cube_ = new LogicalCube<float>(1, 1, oD, 1, driver);
      p_bias_cube_->reset_cube(0.f);
    }
  }
  ~ConvolutionBridge() {
    if (plan_) cct_conv_plan_destroy(plan_);
    delete p_model_cube_; delete p_model_gradient_cube_; delete p_bias_cube_; delete p_bias_gradient_cube_;
  }

  LogicalCube<float>* get_model_cube() { return p_model_cube_; }
  LogicalCube<float>* get_bias_cube() { return p_bias_cube_; }
  LogicalCube<float>* get_model_grad_cube() { return p_model_gradient_cube_; }
  LogicalCube<float>* get_bias_grad_cube() { return p_bias_gradient_cube_; }
  // The scheduler may hand the bridge its own model / bias / gradient storage (ParallelizedBridge_impl.hxx:519-532).
  void set_model_cube(float* p) { p_model_cube_->set_p_data(p); }
  void set_bias_cube(float* p) { if (p_bias_cube_) p_bias_cube_->set_p_data(p); }
  void set_model_grad_cube(float* p) { p_model_gradient_cube_->set_p_data(p); }
  void set_bias_grad_cube(float* p) { if (p_bias_gradient_cube_) p_bias_gradient_cube_->set_p_data(p); }

  void forward() override {
    p_driver->check(cct_conv_forward(plan_, p_input_layer->p_data_cube->get_p_data(), p_model_cube_->get_p_data(),
                                     bias_term ? p_bias_cube_->get_p_data() : nullptr,
                                     p_output_layer->p_data_cube->get_p_data(), fuse_relu ? 1 : 0),
                    "cct_conv_forward");
  }
  // Fold the bridges around this layer into backward(): the ReLU in front of it (input gradient times
  // [input > 0]) and, with pooled_gradient / max_index set, the ReLU + max-pooling bridges behind it (the output
  // gradient is rebuilt from the pooled tensor's gradient instead of being read from p_output_layer).
  bool fuse_relu_backward = false;
  const float* pooled_gradient = nullptr;
  const int32_t* max_index = nullptr;
  int pool_kernel_size = 0, pool_stride = 0;
  void fuse_pool_relu_backward(const float* pooled_grad, const int32_t* index, int kernel_size, int pool_stride_) {
    p_driver->check(cct_conv_plan_reserve_fusion(plan_), "cct_conv_plan_reserve_fusion");
    pooled_gradient = pooled_grad; max_index = index; pool_kernel_size = kernel_size; pool_stride = pool_stride_;
  }

  void backward() override {
    float* dx = needs_to_calc_backward_grad ? p_input_layer->p_gradient_cube->get_p_data() : nullptr;
    float* db = bias_term ? p_bias_gradient_cube_->get_p_data() : nullptr;
    const float* x = p_input_layer->p_data_cube->get_p_data();
    if (!fuse_relu_backward && !pooled_gradient) {
      p_driver->check(cct_conv_backward(plan_, x, p_model_cube_->get_p_data(),
                                        p_output_layer->p_gradient_cube->get_p_data(), dx,
                                        p_model_gradient_cube_->get_p_data(), db),
                      "cct_conv_backward");
      return;
    }
    cct_bwd_fusion f = {nullptr, nullptr, nullptr, 0, 0, fuse_relu_backward ? 1 : 0};
    const float* dy = p_output_layer->p_gradient_cube->get_p_data();
    if (pooled_gradient) {
      f.A = p_output_layer->p_data_cube->get_p_data();
      f.idx = max_index;
      f.dP = pooled_gradient;
      f.pool_k = pool_kernel_size;
      f.pool_s = pool_stride;
      dy = nullptr;
    }
    p_driver->check(cct_conv_backward_fused(plan_, x, p_model_cube_->get_p_data(), dy, &f, dx,
                                            p_model_gradient_cube_->get_p_data(), db),
                    "cct_conv_backward_fused");
  }

 private:
  cct_conv_plan* plan_ = nullptr;
  LogicalCube<float>* p_model_cube_ = nullptr;
  LogicalCube<float>* p_model_gradient_cube_ = nullptr;
  LogicalCube<float>* p_bias_cube_ = nullptr;
  LogicalCube<float>* p_bias_gradient_cube_ = nullptr;
};

// The reference's FullyConnectedBridge (src/bridges/FullyConnectedBridge_impl.hxx:171-235, 257-330): Y = X W^T + b over
// the flattened input, weights [o][d][r][c].  Runs on the C ABI's fully connected plan (three tensor-core GEMMs that read
// X, W and dY in place); feature counts must be multiples of 4.  Output layer: B x num_output x 1 x 1.
class FullyConnectedBridge : public PhysicalOperator {
 public:
  Layer* const p_input_layer;
  Layer* const p_output_layer;
  B200Driver* const p_driver;
  const bool bias_term;
  bool needs_to_calc_backward_grad = true;
  bool fuse_relu = false;           // clamp the output at 0 (the ReLU bridge behind the layer)
  bool fuse_relu_backward = false;  // input gradient times [input > 0] (the ReLU bridge in front)

  FullyConnectedBridge(Layer* in, Layer* out, int num_output, bool bias, B200Driver* driver)
      : p_input_layer(in), p_output_layer(out), p_driver(driver), bias_term(bias),
        in_features_(in->p_data_cube->R * in->p_data_cube->C * in->p_data_cube->D) {
    const LogicalCube<float>* x = in->p_data_cube;
    if (out->p_data_cube->B != x->B || (int)(out->p_data_cube->n_elements / x->B) != num_output)
      driver->check(CCT_ERR_INVALID, "FullyConnectedBridge: output layer must be B x num_output x 1 x 1");
    driver->check(cct_fc_plan_create(driver->ctx(), (int)x->B, (int)in_features_, num_output, bias ? 1 : 0, &plan_),
                  "cct_fc_plan_create");
    p_model_cube_ = new LogicalCube<float>(x->R, x->C, x->D, num_output, driver);
    p_model_gradient_cube_ = new LogicalCube<float>(x->R, x->C, x->D, num_output, driver);
    if (bias) {
      p_bias_cube_ = new LogicalCube<float>(1, 1, num_output, 1, driver);
      p_bias_gradient_cube_ = new LogicalCube<float>(1, 1, num_output, 1, driver);
      p_bias_cube_->reset_cube(0.f);
    }
  }
  ~FullyConnectedBridge() {
    if (plan_) cct_fc_plan_destroy(plan_);
    delete p_model_cube_; delete p_model_gradient_cube_; delete p_bias_cube_; delete p_bias_gradient_cube_;
  }
  LogicalCube<float>* get_model_cube() { return p_model_cube_; }
  LogicalCube<float>* get_bias_cube() { return p_bias_cube_; }
  LogicalCube<float>* get_model_grad_cube() { return p_model_gradient_cube_; }
  LogicalCube<float>* get_bias_grad_cube() { return p_bias_gradient_cube_; }
  void set_model_cube(float* p) { p_model_cube_->set_p_data(p); }
  void set_bias_cube(float* p) { if (p_bias_cube_) p_bias_cube_->set_p_data(p); }
  void set_model_grad_cube(float* p) { p_model_gradient_cube_->set_p_data(p); }
  void set_bias_grad_cube(float* p) { if (p_bias_gradient_cube_) p_bias_gradient_cube_->set_p_data(p); }

  void forward() override {
    p_driver->check(cct_fc_forward(plan_, p_input_layer->p_data_cube->get_p_data(), p_model_cube_->get_p_data(),
                                   bias_term ? p_bias_cube_->get_p_data() : nullptr,
                                   p_output_layer->p_data_cube->get_p_data(), fuse_relu ? 1 : 0, nullptr, 1.f),
                    "cct_fc_forward");
  }
  void backward() override {
    p_driver->check(cct_fc_backward(plan_, p_input_layer->p_data_cube->get_p_data(), p_model_cube_->get_p_data(),
                                    p_output_layer->p_gradient_cube->get_p_data(),
                                    needs_to_calc_backward_grad ? p_input_layer->p_gradient_cube->get_p_data() : nullptr,
                                    p_model_gradient_cube_->get_p_data(),
                                    bias_term ? p_bias_gradient_cube_->get_p_data() : nullptr, fuse_relu_backward ? 1 : 0,
                                    nullptr, 1.f),
                    "cct_fc_backward");
  }

 private:
  size_t in_features_;
  cct_fc_plan* plan_ = nullptr;
  LogicalCube<float>* p_model_cube_ = nullptr;
  LogicalCube<float>* p_model_gradient_cube_ = nullptr;
  LogicalCube<float>* p_bias_cube_ = nullptr;
  LogicalCube<float>* p_bias_gradient_cube_ = nullptr;
};

// The solver fields the updater reads, with the reference's learning-rate policies (src/util.h:76-100).
struct SolverParameter {
  float base_lr = 0.01f, gamma = 0.1f, power = 0.f, momentum = 0.9f, weight_decay = 0.0005f;
  int stepsize = 100000, max_iter = 1;
  std::string lr_policy = "step";
  float learning_rate(float iter) const {
    if (lr_policy == "fixed") return base_lr;
    if (lr_policy == "step") return (float)(base_lr * std::pow((double)gamma, (double)(int)(iter / stepsize)));
    if (lr_policy == "exp") return (float)(base_lr * std::pow((double)gamma, (double)iter));
    if (lr_policy == "inv") return (float)(base_lr * std::pow(1.0 + gamma * iter, -(double)power));
    if (lr_policy == "poly") return (float)(base_lr * std::pow(1.0 - (iter / max_iter), (double)power));
    if (lr_policy == "sigmoid") return (float)(base_lr * (1.0 / (1.0 + std::exp(-gamma * (iter - stepsize)))));
    std::fprintf(stderr, "Unknown learning rate policy: %s\n", lr_policy.c_str());
    std::abort();
  }
};

class SGDGradientUpdater {
 public:
  int current_iter = 0;
  SGDGradientUpdater(size_t n_elements, float* p_model, const SolverParameter* solver, float base_learning_rate,
                     float base_regularization, B200Driver* driver)
      : n_elements_(n_elements), p_model_(p_model), p_solver_(solver), blr_(base_learning_rate),
        br_(base_regularization), p_driver_(driver), history_(n_elements, 1, 1, 1, driver) {
    history_.reset_cube(0.f);
  }
  void set_current_iter(int it) { current_iter = it; }
  float get_stepsize() const { return blr_ * p_solver_->learning_rate((float)current_iter); }
  float get_weight_decay() const { return p_solver_->weight_decay * br_; }
  void update(float* p_gradient) {  // ++iter; g += lambda w; h = lr g + mu h; w -= h
    ++current_iter;
    p_driver_->check(cct_sgd_step(p_driver_->ctx(), n_elements_, p_model_, p_gradient, history_.get_p_data(), get_stepsize(),
                                  p_solver_->momentum, get_weight_decay()),
                     "cct_sgd_step");
  }

 private:
  size_t n_elements_;
  float* p_model_;
  const SolverParameter* p_solver_;
  float blr_, br_;
  B200Driver* p_driver_;
  LogicalCube<float> history_;
};

// The C ABI's communicator: NCCL all-reduce of gradients over the partitions.  Rank 0 calls unique_id() and hands the
// bytes to the other ranks (threads of one process, or processes through any channel); nranks == 1 needs no id.
class Communicator {
 public:
  static std::vector<unsigned char> unique_id() {
    std::vector<unsigned char> id(CCT_COMM_ID_BYTES);
    if (cct_comm_unique_id(id.data()) != CCT_OK) { std::fprintf(stderr, "cct_b200: NCCL is not available\n"); std::abort(); }
    return id;
  }
  Communicator(B200Driver* driver, int nranks, int rank, const unsigned char* id)
      : driver_(driver), nranks_(nranks), rank_(rank) {
    driver->check(cct_comm_init_rank(driver->ctx(), nranks, rank, id, &comm_), "cct_comm_init_rank");
  }
  ~Communicator() { if (comm_) cct_comm_destroy(comm_); }
  Communicator(const Communicator&) = delete;
  int nranks() const { return nranks_; }
  int rank() const { return rank_; }
  void allreduce_sum_begin(float* buf, size_t count) { driver_->check(cct_allreduce_sum_begin(comm_, buf, count), "cct_allreduce_sum_begin"); }
  void wait() { driver_->check(cct_comm_wait(comm_), "cct_comm_wait"); }
  // recv[r * count ...] = rank r's block, on every rank / recv = the sum over ranks of their send[rank * count ...] blocks
  void allgather(const float* send, float* recv, size_t count) { driver_->check(cct_allgather(comm_, send, recv, count), "cct_allgather"); }
  void reduce_scatter_sum(const float* send, float* recv, size_t count) {
    driver_->check(cct_reduce_scatter_sum(comm_, send, recv, count), "cct_reduce_scatter_sum");
  }

 private:
  B200Driver* driver_;
  int nranks_, rank_;
  cct_comm* comm_ = nullptr;
};

// A fully connected layer split over the ranks by output depth: what DeepNet builds as split bridge -> one
// FullyConnectedBridge per GPU over num_output / n outputs, each on the whole mini-batch -> concat bridge
// (src/DeepNet.h:1213-1357), the host round trips of those two bridges replaced by NCCL exchanges.  The layers around
// it stay data parallel: its input and output layers hold this rank's batch slice.
//   forward   all-gather of the input slices -> this rank's output columns for the whole mini-batch -> all-gather of the
//             column slices, of which the rows of this rank's images are put side by side into the output cube;
//   backward  all-gather of the output gradients, this rank's columns of them -> weight / bias gradient of the slice
//             over the whole mini-batch (no sum over ranks is needed: wrap it in a ParallelizedBridgeT without a
//             communicator) and a partial input gradient for every image -> reduce-scatter: each rank receives the sum
//             for its own images (SplitBridge::backward, src/bridges/SplitBridge_impl.hxx:51-90).
// Model and bias cubes are this rank's slice: rows rank * num_output / n ... of the [num_output][in_features] matrix.
class ModelParallelFullyConnectedBridge : public PhysicalOperator {
 public:
  Layer* const p_input_layer;
  Layer* const p_output_layer;
  B200Driver* const p_driver;
  const bool bias_term;
  bool needs_to_calc_backward_grad = true;

  ModelParallelFullyConnectedBridge(Layer* in, Layer* out, int num_output, bool bias, B200Driver* driver, Communicator* comm)
      : p_input_layer(in), p_output_layer(out), p_driver(driver), bias_term(bias), comm_(comm),
        batch_(in->p_data_cube->B), global_batch_(batch_ * comm->nranks()),
        in_features_(in->p_data_cube->R * in->p_data_cube->C * in->p_data_cube->D), outputs_(num_output),
        slice_(check_slice(num_output, comm->nranks(), driver)),
        all_x_(in->p_data_cube->R, in->p_data_cube->C, in->p_data_cube->D, global_batch_, driver),
        all_dx_(in->p_data_cube->R, in->p_data_cube->C, in->p_data_cube->D, global_batch_, driver),
        slice_y_(1, 1, slice_, global_batch_, driver), slice_dy_(1, 1, slice_, global_batch_, driver),
        staging_(1, 1, num_output, global_batch_, driver), all_in_(&all_x_, &all_dx_), slice_out_(&slice_y_, &slice_dy_),
        inner_(&all_in_, &slice_out_, (int)slice_, bias, driver) {
    if (out->p_data_cube->B != batch_ || out->p_data_cube->n_elements / batch_ != outputs_)
      driver->check(CCT_ERR_INVALID, "ModelParallelFullyConnectedBridge: output layer must be B x num_output x 1 x 1");
  }
  LogicalCube<float>* get_model_cube() { return inner_.get_model_cube(); }
  LogicalCube<float>* get_bias_cube() { return inner_.get_bias_cube(); }
  LogicalCube<float>* get_model_grad_cube() { return inner_.get_model_grad_cube(); }
  LogicalCube<float>* get_bias_grad_cube() { return inner_.get_bias_grad_cube(); }
  void set_model_cube(float* p) { inner_.set_model_cube(p); }
  void set_bias_cube(float* p) { inner_.set_bias_cube(p); }
  void set_model_grad_cube(float* p) { inner_.set_model_grad_cube(p); }
  void set_bias_grad_cube(float* p) { inner_.set_bias_grad_cube(p); }
  size_t slice_depth() const { return slice_; }

  void forward() override {
    comm_->allgather(p_input_layer->p_data_cube->get_p_data(), all_x_.get_p_data(), batch_ * in_features_);
    inner_.forward();
    comm_->allgather(slice_y_.get_p_data(), staging_.get_p_data(), global_batch_ * slice_);
    float* y = p_output_layer->p_data_cube->get_p_data();
    for (int q = 0; q < comm_->nranks(); ++q)  // rank q's columns for this rank's images
      copy2d(y + q * slice_, outputs_, staging_.get_p_data() + ((size_t)q * global_batch_ + comm_->rank() * batch_) * slice_,
             slice_, slice_, batch_);
  }
  void backward() override {
    comm_->allgather(p_output_layer->p_gradient_cube->get_p_data(), staging_.get_p_data(), batch_ * outputs_);
    copy2d(slice_dy_.get_p_data(), slice_, staging_.get_p_data() + comm_->rank() * slice_, outputs_, slice_, global_batch_);
    inner_.needs_to_calc_backward_grad = needs_to_calc_backward_grad;
    inner_.backward();
    if (needs_to_calc_backward_grad)
      comm_->reduce_scatter_sum(all_dx_.get_p_data(), p_input_layer->p_gradient_cube->get_p_data(), batch_ * in_features_);
  }

 private:
  static size_t check_slice(int num_output, int nranks, B200Driver* driver) {
    if (nranks < 1 || num_output % nranks)  // "model parallelism must divide depth exactly" (src/DeepNet.h:744-750)
      driver->check(CCT_ERR_INVALID, "ModelParallelFullyConnectedBridge: the ranks must divide num_output");
    return (size_t)(num_output / nranks);
  }
  void copy2d(float* dst, size_t dst_pitch, const float* src, size_t src_pitch, size_t width, size_t rows) {
    p_driver->check(cct_memcpy2d_d2d(p_driver->ctx(), dst, dst_pitch * sizeof(float), src, src_pitch * sizeof(float),
                                     width * sizeof(float), rows), "cct_memcpy2d_d2d");
  }
  Communicator* comm_;
  size_t batch_, global_batch_, in_features_, outputs_, slice_;
  LogicalCube<float> all_x_, all_dx_, slice_y_, slice_dy_, staging_;
  Layer all_in_, slice_out_;
  FullyConnectedBridge inner_;
};

// One batch partition on one GPU.  forward()/backward() run the sub-bridge; backward() then sums the model and bias
// gradients over all partitions (`comm`, NULL: single partition) and applies the SGD update, identical on every
// partition.  Model and bias (and their gradients) are contiguous (W | bias) so one all-reduce covers both.
// SubBridge: ConvolutionBridge or FullyConnectedBridge.
template <class SubBridge>
class ParallelizedBridgeT : public PhysicalOperator {
 public:
  ParallelizedBridgeT(SubBridge* sub, const SolverParameter* solver, B200Driver* driver, Communicator* comm = nullptr,
                      float model_lr_mult = 1.f, float model_decay_mult = 1.f, float bias_lr_mult = 2.f,
                      float bias_decay_mult = 0.f)
      : sub_(sub), p_driver_(driver), comm_(comm), n_w_(sub->get_model_cube()->n_elements),
        n_b_(sub->bias_term ? sub->get_bias_cube()->n_elements : 0), params_(n_w_ + n_b_, 1, 1, 1, driver),
        grads_(n_w_ + n_b_, 1, 1, 1, driver),
        p_grad_updater(n_w_, params_.get_p_data(), solver, model_lr_mult, model_decay_mult, driver),
        p_grad_updater_bias(n_b_ ? n_b_ : 1, params_.get_p_data() + n_w_, solver, bias_lr_mult, bias_decay_mult, driver) {
    sub->set_model_cube(params_.get_p_data());
    sub->set_model_grad_cube(grads_.get_p_data());
    sub->set_bias_cube(params_.get_p_data() + n_w_);
    sub->set_bias_grad_cube(grads_.get_p_data() + n_w_);
  }
  bool update_model_gradients = true;
  void set_update_model_gradients(bool v) { update_model_gradients = v; }
  LogicalCube<float>* get_model_cube() { return sub_->get_model_cube(); }
  LogicalCube<float>* get_bias_cube() { return sub_->get_bias_cube(); }
  float* get_model_gradient_device() { return grads_.get_p_data(); }
  void forward() override { sub_->forward(); }
  void backward() override {
    sub_->backward();
    if (comm_) {
      comm_->allreduce_sum_begin(grads_.get_p_data(), n_w_ + n_b_);  // gradients are summed, not averaged (:916-955)
      comm_->wait();
    }
    if (!update_model_gradients) return;
    p_grad_updater.update(grads_.get_p_data());
    if (n_b_) p_grad_updater_bias.update(grads_.get_p_data() + n_w_);
  }

 private:
  SubBridge* sub_;
  B200Driver* p_driver_;
  Communicator* comm_;
  size_t n_w_, n_b_;
  LogicalCube<float> params_, grads_;

 public:
  SGDGradientUpdater p_grad_updater, p_grad_updater_bias;
};
typedef ParallelizedBridgeT<ConvolutionBridge> ParallelizedBridge;

}  // namespace cct
