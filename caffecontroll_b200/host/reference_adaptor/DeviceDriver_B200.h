// B200Driver: the device driver a Caffe con Troll maintainer adds next to CPUDriver / GPUDriver
// (src/sched/DeviceDriver_CPU.h, DeviceDriver_GPU.h).  It derives from the reference's own DeviceDriver
// (src/sched/DeviceDriver.h:56-274), implements every pure virtual, and forwards to the C ABI of cct_b200.h.
// This header only compiles inside the reference tree (include path: <reference>/src and <this repo>/include).
//
// What a bridge needs from a driver splits in two here:
//   * memory, copies, fills, saxpy / saxpby for the SGD updater: implemented below through cct_* calls;
//   * the per-image lowering / GEMM / bias / pooling entry points GPUDriver offers (lower_cube, sgemm,
//     inverse_lower_cube, forward_bias, ...): NOT used by the B200 bridges - a whole bridge pass is one C-ABI call
//     (cct_conv_forward / cct_conv_backward) - so sgemm and the generic maps report an error if something calls them.
// Errors follow the reference's convention: print, then assert(false) (src/sched/DeviceDriver.h:48-51).
#ifndef _DEVICE_DRIVER_B200_H
#define _DEVICE_DRIVER_B200_H

#include <deque>
#include <iostream>

#include "sched/DeviceDriver.h"
#include "cct_b200.h"

class B200Driver : public DeviceDriver {
public:
  int gpu_id;

  explicit B200Driver(int _gpu_id = 0) : gpu_id(_gpu_id), ctx_(NULL) { check(cct_ctx_create(gpu_id, &ctx_), "cct_ctx_create"); }
  ~B200Driver() {
    for (size_t i = 0; i < pointers_.size(); ++i) delete pointers_[i];
    if (ctx_) cct_ctx_destroy(ctx_);
  }

  cct_ctx * ctx() const { return ctx_; }

  // The reference's GPUDriver leaks one DeviceMemoryPointer per call (src/sched/DeviceDriver_GPU.cu:849-852); here the
  // driver keeps them and frees them with itself.
  DeviceMemoryPointer * get_device_pointer(void * ptr, size_t size_in_byte) {
    pointers_.push_back(new DeviceMemoryPointer_Local_GPURAM(gpu_id, ptr, size_in_byte));
    return pointers_.back();
  }
  void * choose_ptr(void * host, void * device) { return device; }

  void malloc(DeviceMemoryPointer * dst) { check(cct_malloc(ctx_, dst->size_in_byte, &dst->ptr), "cct_malloc"); }
  void free(DeviceMemoryPointer * dst) { check(cct_free(ctx_, dst->ptr), "cct_free"); }
  // Host pointers are DEVICEMEMORY_LOCAL_RAM (CPUDriver::get_device_pointer), everything else is on this GPU;
  // the call returns when the copy has landed, as GPUDriver::memcpy (cudaMemcpy) does.
  void memcpy(DeviceMemoryPointer * dst, DeviceMemoryPointer * src) {
    if (src->type == DEVICEMEMORY_LOCAL_RAM) check(cct_memcpy_h2d(ctx_, dst->ptr, src->ptr, dst->size_in_byte), "cct_memcpy_h2d");
    else if (dst->type == DEVICEMEMORY_LOCAL_RAM) check(cct_memcpy_d2h(ctx_, dst->ptr, src->ptr, dst->size_in_byte), "cct_memcpy_d2h");
    else check(cct_memcpy_d2d(ctx_, dst->ptr, src->ptr, dst->size_in_byte), "cct_memcpy_d2d");
    device_sync();
  }
  void memset(DeviceMemoryPointer * dst, const char value) { check(cct_memset(ctx_, dst->ptr, value, dst->size_in_byte), "cct_memset"); }

  // y = alpha x + y and y = alpha x + beta y on device vectors (the SGD updater's calls, src/algorithms/GradientUpdater.h:163-181)
  void math_saxpy(const float alpha, DeviceMemoryPointer * X, DeviceMemoryPointer * Y) const {
    check(cct_saxpby(ctx_, X->size_in_byte / sizeof(float), alpha, (const float *) X->ptr, 1.f, (float *) Y->ptr), "cct_saxpby");
  }
  void math_saxpby(const float alpha, DeviceMemoryPointer * X, const float beta, DeviceMemoryPointer * Y) const {
    check(cct_saxpby(ctx_, X->size_in_byte / sizeof(float), alpha, (const float *) X->ptr, beta, (float *) Y->ptr), "cct_saxpby");
  }
  void math_saxpy(const int nElements, const float alpha, float * X, float * Y) const {
    check(cct_saxpby(ctx_, nElements, alpha, X, 1.f, Y), "cct_saxpby");
  }
  void math_saxpby(const int nElements, const float alpha, const float * X, const float beta, float * Y) const {
    check(cct_saxpby(ctx_, nElements, alpha, X, beta, Y), "cct_saxpby");
  }
  void L1_update(const int n_elements, float * const p_gradient, const float lambda, const float * const p_model) {
    check(cct_l1_update(ctx_, n_elements, p_gradient, lambda, p_model), "cct_l1_update");
  }
  void set_num_threads(const int nThreads) {}
  void sgemm(const enum CBLAS_ORDER order, CBLAS_TRANSPOSE TA, CBLAS_TRANSPOSE TB, int M, int N, int K, float alpha,
             float * pA, int LDA, float * pB, int LDB, float beta, float * pC, int LDC) {
    std::cerr << "B200Driver::sgemm: the B200 bridges run whole passes through cct_conv_* / cct_fc_*; "
                 "no bridge should reach the per-image GEMM entry point" << std::endl;
    assert(false);
  }

  // Fillers (src/sched/DeviceDriver_CPU.cpp:661-707): same generators as the CPU driver, results uploaded.
  void sconstant_initialize(DeviceMemoryPointer * arr, const float value) {
    check(cct_fill_f32(ctx_, (float *) arr->ptr, arr->size_in_byte / sizeof(float), value), "cct_fill_f32");
  }
  void sgaussian_initialize(DeviceMemoryPointer * arr, const float mean, const float std_dev, const int random_seed = -1) {
    check(cct_fill_random(ctx_, (float *) arr->ptr, arr->size_in_byte / sizeof(float), CCT_FILL_GAUSSIAN, mean, std_dev, random_seed),
          "cct_fill_random");
  }
  void sinitialize_xavier(DeviceMemoryPointer * arr, const size_t n_batch, const int random_seed = -1) {
    const size_t n = arr->size_in_byte / sizeof(float);
    check(cct_fill_random(ctx_, (float *) arr->ptr, n, CCT_FILL_XAVIER, (float) (n / n_batch), 0.f, random_seed), "cct_fill_random");
  }
  void sbernoulli_initialize(DeviceMemoryPointer * arr, const float p, const int random_seed = -1) {
    check(cct_fill_random(ctx_, (float *) arr->ptr, arr->size_in_byte / sizeof(float), CCT_FILL_BERNOULLI, p, 0.f, random_seed),
          "cct_fill_random");
  }

  void device_sync() { check(cct_sync(ctx_), "cct_sync"); }
  void set_device_id(int id) { assert(id == gpu_id); }  // a context is bound to its device at construction

  void check(int rc, const char * what) const {
    if (rc != CCT_OK) {
      std::cout << "B200Driver: " << what << " failed (code " << rc << "): " << (ctx_ ? cct_last_error_string(ctx_) : "") << std::endl;
      assert(false);
    }
  }

private:
  cct_ctx * ctx_;
  std::deque<DeviceMemoryPointer *> pointers_;
};

#endif
