/* cct_b200.h — C ABI of the B200 (sm_100a) convolution hot path for Caffe con Troll.
 *
 * This is the drop-in boundary: everything above it (the C++ bridge mirror in caffecontroll_b200/host/, the
 * Python binding in caffecontroll_b200/capi.py, or a DeviceDriver subclass inside the reference tree) speaks
 * plain pointers and sizes.  All tensors are fp32, NCHW, dense — the layout of the reference's
 * LogicalCube<float, Layout_CRDB> (src/LogicalCube_impl.hxx:217-219).  Unless a function says "host", every
 * data pointer is a device pointer on the context's device, owned by the caller.
 *
 * Every function returns CCT_OK (0) or a CCT_ERR_* code and never aborts; the reference's convention
 * ("functions return void, on error assert(false)", src/sched/DeviceDriver.h:48-51) is re-created by the
 * bridge adaptor on top.  Work is enqueued on the context's stream; cct_sync() waits for it and reports
 * device-side failures (a bounded wait that ran out).  A context may be used from any host thread, one
 * caller at a time (the reference runs each bridge call on a fresh std::thread: src/bridges/PhysicalStratum.h:43-70).
 */
#ifndef CCT_B200_H
#define CCT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  CCT_OK = 0,
  CCT_ERR_INVALID = 1,     /* bad argument / shape */
  CCT_ERR_CUDA = 2,        /* a CUDA runtime call failed; see cct_last_error_string */
  CCT_ERR_NOMEM = 3,
  CCT_ERR_TIMEOUT = 4,     /* a bounded device-side wait gave up */
  CCT_ERR_UNSUPPORTED = 5
};

/* Which arithmetic runs the three contractions. */
enum {
  CCT_ALGO_AUTO = 0,       /* tcgen05 3xTF32 where the shape allows, else SIMT fp32 */
  CCT_ALGO_SIMT_FP32 = 1,  /* direct convolution in fp32 FMA (exact fp32 products) */
  CCT_ALGO_UMMA_3XTF32 = 2 /* implicit GEMM on tcgen05/TMEM, each operand split hi+lo in TF32, 3 MMAs */
};

typedef struct cct_ctx cct_ctx;
typedef struct cct_conv_plan cct_conv_plan;

/* ---- context, memory, sync: replaces DeviceDriver::{malloc,free,memcpy,memset,device_sync,set_device_id}
 *      (src/sched/DeviceDriver.h:56-120) and GPUDriver's per-call cublasCreate/Destroy
 *      (src/sched/DeviceDriver_GPU.cu:1601-1620): a context is created once and reused. ---- */
int cct_ctx_create(int device_id, cct_ctx** out);
/* Same, but enqueue on a stream the caller owns (a cudaStream_t passed as void*; NULL = legacy default stream). */
int cct_ctx_create_on_stream(int device_id, void* cuda_stream, cct_ctx** out);
int cct_ctx_destroy(cct_ctx* ctx);
int cct_sync(cct_ctx* ctx);
const char* cct_last_error_string(cct_ctx* ctx);
int cct_device_count(int* count);

int cct_malloc(cct_ctx* ctx, size_t bytes, void** dptr);
int cct_free(cct_ctx* ctx, void* dptr);
int cct_malloc_host(cct_ctx* ctx, size_t bytes, void** hptr); /* pinned host memory */
int cct_free_host(cct_ctx* ctx, void* hptr);
int cct_memcpy_h2d(cct_ctx* ctx, void* dst, const void* src, size_t bytes); /* stream-ordered */
int cct_memcpy_d2h(cct_ctx* ctx, void* dst, const void* src, size_t bytes); /* stream-ordered */
int cct_memcpy_d2d(cct_ctx* ctx, void* dst, const void* src, size_t bytes);
/* `rows` runs of width_bytes each, the runs dst_pitch / src_pitch bytes apart (stream-ordered, device to device): the
 * column blocks a model-parallel layer's concat and split bridges move (src/bridges/ConcatBridge_impl.hxx,
 * src/bridges/SplitBridge_impl.hxx copy whole cubes; here the slices sit side by side in one row-major cube). */
int cct_memcpy2d_d2d(cct_ctx* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                     size_t rows);
int cct_memset(cct_ctx* ctx, void* dptr, int byte_value, size_t bytes);
/* DeviceDriver::sconstant_initialize (src/sched/DeviceDriver.h:236, DeviceDriver_GPU.cu:1189-1200). */
int cct_fill_f32(cct_ctx* ctx, float* dptr, size_t count, float value);
/* The weight / bias fillers a bridge constructor applies (ConvolutionBridge::initialize_logical_cube,
 * src/bridges/ConvolutionBridge_impl.hxx:250-267; CPUDriver::sgaussian_initialize, sinitialize_xavier,
 * sbernoulli_initialize, src/sched/DeviceDriver_CPU.cpp:661-699): std::mt19937(seed) feeding the standard
 * distributions on the host, uploaded to dptr; seed == -1 takes a random seed (solver.random_seed's default).
 *   CCT_FILL_GAUSSIAN : a = mean, b = std            CCT_FILL_XAVIER : a = fan_in (elements / n_batch), uniform in
 *   +-sqrt(3 / fan_in)                               CCT_FILL_BERNOULLI : a = p
 * With the same C++ standard library the values equal the reference's for the same seed ("constant" is cct_fill_f32). */
enum { CCT_FILL_GAUSSIAN = 0, CCT_FILL_XAVIER = 1, CCT_FILL_BERNOULLI = 2 };
int cct_fill_random(cct_ctx* ctx, float* dptr, size_t count, int kind, float a, float b, long seed);

/* ---- the convolution bridge: replaces ConvolutionBridge::forward/backward
 *      (src/bridges/ConvolutionBridge_impl.hxx:294-500, 551-773) together with the driver entry points they
 *      call: lower_cube, sgemm, forward_bias, backward_bias, inverse_lower_cube
 *      (src/sched/DeviceDriver.h:122-190; GPU versions src/sched/DeviceDriver_GPU.cu:205-228, 670-786, 1059-1139)
 *      and Connector::remap_output (src/Connector_impl_Lowering_type1.hxx:92-128), which has no counterpart
 *      here because outputs are produced directly in [b][o][r][c] order. ---- */
typedef struct cct_conv_desc {
  int batch;      /* B: images per call (one partition of the mini-batch) */
  int in_depth;   /* D */
  int in_size;    /* n: square input, as the reference requires (src/sched/DeviceDriver_CPU.cpp:137-140) */
  int out_depth;  /* o: number of filters */
  int kernel;     /* k */
  int stride;     /* s */
  int pad;        /* p */
  int groups;     /* g: D and o must be multiples of g; filter tensor is [o][D/g][k][k] */
  int bias_term;  /* 0: no bias (bias/db pointers ignored) */
  int algo;       /* CCT_ALGO_* */
} cct_conv_desc;

int cct_conv_plan_create(cct_ctx* ctx, const cct_conv_desc* desc, cct_conv_plan** out);
int cct_conv_plan_destroy(cct_conv_plan* plan);
/* m = (n + 2p - k)/s + 1 (src/DeepNet.h:112-115). */
int cct_conv_out_size(const cct_conv_desc* desc, int* out_size);
/* The algorithm the plan resolved to (CCT_ALGO_SIMT_FP32 or CCT_ALGO_UMMA_3XTF32). */
int cct_conv_plan_algo(const cct_conv_plan* plan, int* algo);
/* Bytes of scratch memory the plan owns (packed weight splits, split-K partial sums). */
int cct_conv_plan_workspace_bytes(const cct_conv_plan* plan, size_t* bytes);

/* Y[b][o][r][c] = bias[o] + sum_{d,kr,kc} W[o][d][kr][kc] * X[b][d][r*s-p+kr][c*s-p+kc]   (zero outside X).
 * relu != 0 additionally clamps Y at 0 (the ReLU bridge that follows every CaffeNet convolution,
 * src/kernels/relu.hxx:17-26, folded into the epilogue). */
int cct_conv_forward(cct_conv_plan* plan, const float* X, const float* W, const float* bias, float* Y, int relu);

/* dW, db are overwritten (beta = 0, src/bridges/ConvolutionBridge_impl.hxx:619-621); dX is written only when
 * dX != NULL (needs_to_calc_backward_grad, src/bridges/AbstractBridge.h; the first convolution of a net skips it,
 * src/DeepNet.h:1108-1110).  dY is not modified (the reference's CPU path permutes it in place, :604). */
int cct_conv_backward(cct_conv_plan* plan, const float* X, const float* W, const float* dY, float* dX, float* dW,
                      float* db);

/* cct_conv_backward with the backward passes of the neighbouring bridges folded in (the reference runs them as
 * separate bridges: MaxPoolingBridge::backward src/bridges/MaxPoolingBridge_impl.hxx:106-151, ReLUBridge::backward
 * src/bridges/ReLUBridge_impl.hxx:65-99).
 *   - Output side.  With f->dP != NULL the gradient of this layer's output is not taken from dY (pass NULL) but built
 *     from what sits behind the convolution, conv -> ReLU -> max-pool(pool_k, pool_s):
 *         dY = (A > 0) * maxpool_backward(dP, idx)
 *     A = this layer's forward output [batch][out_depth][m][m] (pre- or post-ReLU: only its sign is used), idx = the
 *     int32 indices cct_maxpool_forward wrote, dP = gradient of the pooled tensor.  One HBM-bound pass into
 *     plan-owned scratch (cct_conv_plan_reserve_fusion) feeds both gradient kernels.  If P, the pooled tensor
 *     cct_maxpool_forward wrote, is given as well (or instead of A), the sign is taken from it - the element a window
 *     points at holds that window's maximum, so the result is bit-identical - and A, (m / pooled size)^2 times larger,
 *     is not read.
 *   - Input side.  relu_mask_dx != 0 writes dX * [X > 0] instead of dX: the ReLU bridge in front of this layer (whose
 *     output X is), applied by one streaming pass right behind the data-gradient kernel.
 * f == NULL behaves like cct_conv_backward. */
typedef struct cct_bwd_fusion {
  const float* A;
  const int32_t* idx;
  const float* dP;
  int pool_k, pool_s;
  int relu_mask_dx;
  const float* P; /* optional, see above; NULL = take the sign from A */
} cct_bwd_fusion;
int cct_conv_backward_fused(cct_conv_plan* plan, const float* X, const float* W, const float* dY,
                            const cct_bwd_fusion* f, float* dX, float* dW, float* db);
/* Allocates the plan-owned buffer (one tensor of the layer's output size) that cct_conv_backward_fused fills when it
 * is given a pooled gradient.  Call it once, next to cct_conv_plan_create, for every plan that will be used that way:
 * cct_conv_backward_fused itself never allocates and returns CCT_ERR_INVALID if the buffer is missing. */
int cct_conv_plan_reserve_fusion(cct_conv_plan* plan);

/* Host-buffer forms of the two calls above, for callers that keep cubes in host memory as the reference's
 * ParallelizedBridge does (src/bridges/ParallelizedBridge_impl.hxx:538-671, 686-738, 779-830, 895-910,
 * 1071-1122): inputs are copied to plan-owned device buffers, the kernels run, results are copied back, and the
 * call returns after the results have landed.  Pinned host memory (cct_malloc_host) makes the copies asynchronous;
 * batches of sixteen images or more move in eight slices on two side streams, so that the upload of one slice, the
 * kernels of the previous one and the download of the one before overlap.
 * cct_conv_backward_host accepts hX == NULL and/or hW == NULL, meaning "the copy staged by the last
 * cct_conv_forward_host on this plan" (the reference keeps the input cube on the device between the two passes). */
int cct_conv_forward_host(cct_conv_plan* plan, const float* hX, const float* hW, const float* hbias, float* hY,
                          int relu);
int cct_conv_backward_host(cct_conv_plan* plan, const float* hX, const float* hW, const float* hdY, float* hdX,
                           float* hdW, float* hdb);

/* The weight and bias gradient of cct_conv_backward for callers that must not allocate device memory at the point
 * of the call.  No counterpart in the reference.  Who needs it: code running where a cudaMalloc would fail or stall —
 * under a memory pool that already owns the whole device, inside a latency-critical section, or in a process whose
 * allocator hooks forbid late allocations.  Such a caller cannot create a cct_conv_plan (a plan allocates its tables
 * and split-K scratch), so this call takes the layer description directly and keeps its scratch (the lowered-matrix
 * row table and the split partial sums) in a 16 MiB array that is part of the library image on every device that
 * loads it.  It calls no cudaMalloc / cudaFree and no allocating library routine; X, dY, dW, db are the caller's
 * device buffers as in cct_conv_backward (dW, db overwritten; db ignored without bias_term).
 *   - Limit: the row table plus one split's partial sums must fit in 16 MiB, else CCT_ERR_UNSUPPORTED with the needed
 *     size in cct_last_error_string.  The pixel range is cut into the same bounded accumulation chains as in the
 *     plan-based path (at most 176 blocks of 32 pixels per partial sum); when the array cannot hold all the splits at
 *     once they are processed in rounds that reuse the slices, each round's reduction adding to dW / db.
 *   - The 16 MiB come into being when the library's device code is first loaded on a device, which with lazy module
 *     loading can be this call itself.  Make one call of it (or any plan-based convolution call) on every device
 *     BEFORE the pool takes the device or the no-allocation section starts; a failure at that point surfaces as
 *     CCT_ERR_NOMEM or CCT_ERR_CUDA from this function.  The same first call looks up the array's device address
 *     (cudaGetSymbolAddress) and should precede any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's contents (nothing in it needs to
 *     start at zero: every slot that is read is written first by the same call).  Two calls that overlap on the GPU -
 *     different streams or contexts of the same device - race on it; serialise them.
 * Results equal cct_conv_backward's dW, db up to the rounding of a different split count; both hold the 1e-4
 * tolerance against the CPU path at the BASELINE sizes (tests/test_zz_no_alloc.py). */
int cct_conv_weight_grad_noalloc(cct_ctx* ctx, const cct_conv_desc* desc, const float* X, const float* dY, float* dW,
                                 float* db);

/* Per-kernel device times of the plan's most recent forward and backward call, for measurement: when enabled,
 * CUDA events are recorded around each kernel group on the context's stream.  ms[0] forward contraction,
 * ms[1] weight(+bias)-gradient contraction, ms[2] its split reduction, ms[3] data-gradient contraction(s),
 * ms[4] weight repacking (all calls).  The getter synchronises the stream.  No counterpart in the reference
 * (its Report objects hold host wall-clock: src/Report.h:13-91). */
int cct_conv_plan_enable_timing(cct_conv_plan* plan, int enable);
int cct_conv_plan_last_timings(cct_conv_plan* plan, float ms[5]);

/* ---- the fully connected bridge: replaces FullyConnectedBridge::forward/backward
 *      (src/bridges/FullyConnectedBridge_impl.hxx:171-235, 257-330) and the driver calls they make (sgemm_new,
 *      backward_bias_fc: src/sched/DeviceDriver_GPU.cu:1142-1160).  X is [batch][in_features] (a cube of any R x C x D
 *      with R*C*D = in_features, flattened as the reference does), W is [out_features][in_features], Y is
 *      [batch][out_features].  in_features and out_features must be multiples of 4.  The three contractions run as
 *      3xTF32 on the tensor cores with the operands read in place by TMA (nothing is transposed or packed). ---- */
typedef struct cct_fc_plan cct_fc_plan;
int cct_fc_plan_create(cct_ctx* ctx, int batch, int in_features, int out_features, int bias_term, cct_fc_plan** out);
int cct_fc_plan_destroy(cct_fc_plan* plan);
int cct_fc_plan_workspace_bytes(const cct_fc_plan* plan, size_t* bytes);
/* Y = X * W^T + bias.  relu != 0 clamps at 0 (the ReLU bridge behind the layer); drop_mask != NULL then multiplies by
 * (mask != 0) * drop_scale (DropoutBridge::forward in training, src/bridges/DropoutBridge_impl.hxx:71-74: the mask
 * holds one unsigned int per output element, drop_scale = 1 / (1 - dropout_ratio)). */
int cct_fc_forward(cct_fc_plan* plan, const float* X, const float* W, const float* bias, float* Y, int relu,
                   const uint32_t* drop_mask, float drop_scale);
/* dW = dY^T * X and db = column sums of dY (both overwritten); dX = dY * W when dX != NULL.  The bridges in front of the
 * layer can be folded into dX: in_drop_mask != NULL multiplies dX by (mask != 0) * in_drop_scale (DropoutBridge::backward),
 * in_relu != 0 by [X > 0] (ReLUBridge::backward; X is this layer's input, i.e. the output of those bridges). */
int cct_fc_backward(cct_fc_plan* plan, const float* X, const float* W, const float* dY, float* dX, float* dW, float* db,
                    int in_relu, const uint32_t* in_drop_mask, float in_drop_scale);
/* Per-kernel-group device times of the most recent calls (as cct_conv_plan_last_timings): ms[0] forward, ms[1] weight
 * and bias gradient, ms[3] data gradient. */
int cct_fc_plan_enable_timing(cct_fc_plan* plan, int enable);
int cct_fc_plan_last_timings(cct_fc_plan* plan, float ms[5]);

/* Failure-path self-test (no counterpart in the reference, whose kernels never wait on anything): launches one warp
 * that waits, through the same bounded wait the convolution kernels use, on a barrier nothing completes, with a limit
 * of `limit_cycles` SM clock cycles (at most the kernels' own limit).  The wait runs out, the kernel returns normally,
 * and the next cct_sync on the context reports CCT_ERR_TIMEOUT and clears the status word; calls made after that run
 * as usual.  Nothing traps or faults. */
int cct_selftest_bounded_wait(cct_ctx* ctx, long long limit_cycles);

/* ---- adjacent layers whose backward masks feed the convolution backward ---- */
/* DeviceDriver::maxpool_forward / maxpool_backward (src/sched/DeviceDriver_CPU.cpp:369-421): windows k x k,
 * stride s, no padding, clipped at the border, output size (n-k)/s+1 by floor; idx = int32 offset h*n+w of the
 * first maximum inside the (n x n) plane; backward zero-fills dX and adds dY at idx. */
int cct_maxpool_forward(cct_ctx* ctx, const float* X, float* Y, int32_t* idx, int planes, int n, int k, int s);
int cct_maxpool_backward(cct_ctx* ctx, const float* dY, const int32_t* idx, float* dX, int planes, int n, int k,
                         int s);
/* ReLU bridge (src/kernels/relu.hxx:17-43). */
int cct_relu_forward(cct_ctx* ctx, const float* X, float* Y, size_t count);
int cct_relu_backward(cct_ctx* ctx, const float* X, const float* dY, float* dX, size_t count);
/* ReLUBridge::backward after MaxPoolingBridge::backward in one pass: given the convolution output A (pre- or
 * post-ReLU: only its sign is used), the pooling indices and the gradient of the pooled tensor,
 *   dA[plane][h][w] = (A > 0) * sum over windows (ph,pw) covering (h,w) with idx == h*n+w of dP[plane][ph][pw]. */
int cct_pool_relu_backward(cct_ctx* ctx, const float* A, const int32_t* idx, const float* dP, float* dA, int planes,
                           int n, int k, int s);

/* ---- gradient summation across the partitions of the mini-batch: replaces the device-to-host gather and the serial
 *      host-side sum of ParallelizedBridge::backward (src/bridges/ParallelizedBridge_impl.hxx:876-971) by an NCCL
 *      all-reduce(SUM, fp32) over NVLink.  One communicator per context (= per GPU / rank); NCCL is loaded at run time
 *      the first time a communicator of more than one rank is created.  Rank 0 obtains an id with cct_comm_unique_id and
 *      hands its bytes to every rank by whatever channel the launcher offers (a file, MPI, a TCP store); every rank then
 *      calls cct_comm_init_rank (collective: it returns once all ranks have joined).
 *      cct_allreduce_sum_begin orders the reduction behind the work already queued on the context's stream and runs it
 *      on the communicator's own stream, so that kernels enqueued afterwards (the backward pass of the layers below)
 *      overlap it; cct_comm_wait makes the context's stream wait for every reduction begun so far - call it before the
 *      SGD step that reads the buffers.  cct_allreduce_sum = begin + wait.  nranks == 1 makes all of them no-ops.
 *      Between the first begin and the wait the library's persistent kernels size their grids for eight SMs fewer,
 *      the ones NCCL's CTAs occupy; cct_comm_init_rank sets NCCL_MAX_CTAS=8 in the process environment for that unless
 *      the variable is already set (a few CTAs carry a reduction at NVLink speed).  Create the communicator before the
 *      layer plans: plans made afterwards choose their split counts and tilings for the SMs that remain. ---- */
#define CCT_COMM_ID_BYTES 128
typedef struct cct_comm cct_comm;
int cct_comm_unique_id(unsigned char id[CCT_COMM_ID_BYTES]);
int cct_comm_init_rank(cct_ctx* ctx, int nranks, int rank, const unsigned char id[CCT_COMM_ID_BYTES], cct_comm** out);
int cct_comm_destroy(cct_comm* comm);
int cct_comm_size(const cct_comm* comm, int* nranks, int* rank);
int cct_allreduce_sum_begin(cct_comm* comm, float* buf, size_t count);
int cct_comm_wait(cct_comm* comm);
int cct_allreduce_sum(cct_comm* comm, float* buf, size_t count);
/* The exchanges of a model-parallel fully connected layer (DeepNet builds it as split bridge -> one fully connected
 * bridge per GPU over an equal slice of the output depth -> concat bridge, with the whole mini-batch copied to every
 * GPU through the host: src/DeepNet.h:1213-1357).  cct_allgather: recv[r * count_per_rank ...] = rank r's send block,
 * for every rank r (ncclAllGather).  cct_reduce_scatter_sum: recv = the sum over ranks of their
 * send[rank * count_per_rank ...] blocks (ncclReduceScatter) - the sum the split bridge's backward pass forms of the
 * slices' input gradients.  Both are ordered behind the work queued on the context's stream and the context's stream
 * waits for them; with one rank they are copies. */
int cct_allgather(cct_comm* comm, const float* send, float* recv, size_t count_per_rank);
int cct_reduce_scatter_sum(cct_comm* comm, const float* send, float* recv, size_t count_per_rank);

/* ---- the other bridges of a CaffeNet iteration, as HBM-bound kernels ---- */
/* LRNBridge (across channels; src/bridges/LRNBridge_impl.hxx:46-190, src/kernels/lrn.hxx:38-180, exact pow as in the
 * reference's test build): scale = 1 + (alpha / local_size) * sum over the local_size channels around d of X^2,
 * Y = X / scale^beta.  X, Y, scale, dY, dX are [batch][depth][plane] with plane = R * C; local_size is odd.
 * `scale` is the bridge's denominator cube.  It may be NULL in both calls: the forward pass then does not store it and
 * the backward pass forms it again from X (windows of 3 and 5 channels; other windows need Y and scale of the forward
 * pass and answer CCT_ERR_UNSUPPORTED without them).  For windows of 3 and 5 channels the backward pass does not read
 * Y (it may be NULL): Y = X / scale^beta is formed again as the forward pass formed it. */
int cct_lrn_forward(cct_ctx* ctx, const float* X, float* Y, float* scale, int batch, int depth, int plane, int local_size,
                    float alpha, float beta);
int cct_lrn_backward(cct_ctx* ctx, const float* X, const float* Y, const float* scale, const float* dY, float* dX,
                     int batch, int depth, int plane, int local_size, float alpha, float beta);
/* DropoutBridge in training, forward and backward alike (src/bridges/DropoutBridge_impl.hxx:71-74):
 * out = in * (mask != 0) * scale, one unsigned int of mask per element, scale = 1 / (1 - dropout_ratio).  The mask is
 * the caller's (the reference draws it on the host, src/bridges/DropoutBridge_impl.hxx:62-66); in == out is allowed. */
int cct_dropout_apply(cct_ctx* ctx, const float* in, const uint32_t* mask, float scale, float* out, size_t count);
/* Draws a mask on the device: element i is 1 with probability 1 - ratio (as GPUDriver::rand_uint_initialize followed by
 * the threshold test does, src/bridges/DropoutBridge_impl.hxx:100-104).  Counter-based: (seed, call) fixes the mask,
 * whatever the launch shape; use a new `call` value every iteration. */
int cct_dropout_mask(cct_ctx* ctx, uint32_t* mask, size_t count, float ratio, uint64_t seed, uint64_t call);
/* SoftmaxLossBridge (src/kernels/softmax.hxx:17-80; host-only in the reference): prob[b][c] = softmax of X[b][:],
 * *loss = sum over images of -log(max(prob[b][label], FLT_MIN)) (image_loss: `batch` floats of scratch that receive
 * the per-image terms).  labels holds one float per image, as the reference's label cube does.  The backward pass
 * writes dX = (prob - onehot(label)) * scale; the reference uses scale = 1 / batch (with data parallelism: the batch
 * of the whole job, so that the partitions' gradients add up). */
int cct_softmax_loss_forward(cct_ctx* ctx, const float* X, const float* labels, float* prob, float* image_loss,
                             float* loss, int batch, int classes);
int cct_softmax_loss_backward(cct_ctx* ctx, const float* prob, const float* labels, float* dX, int batch, int classes,
                              float scale);

/* ---- parameter update: SGDGradientUpdater::update (src/algorithms/GradientUpdater.h:154-193) as one kernel:
 *      g += lambda*w (if lambda != 0);  h = lr*g + momentum*h;  w -= h. ---- */
int cct_sgd_step(cct_ctx* ctx, size_t count, float* w, float* g, float* h, float lr, float momentum, float lambda);
/* y = alpha * x + beta * y on device vectors: DeviceDriver::math_saxpy (beta = 1) and math_saxpby
 * (src/sched/DeviceDriver.h:197-206), the calls the reference's SGDGradientUpdater makes when it is instantiated on a
 * device driver unchanged. */
int cct_saxpby(cct_ctx* ctx, size_t count, float alpha, const float* x, float beta, float* y);
/* g += lambda * sign(w), sign(0) = -1: DeviceDriver::L1_update (src/sched/DeviceDriver.h:114-117,
 * src/sched/DeviceDriver_CPU.cpp:111-117), the updater's step for regularization_type "L1"; follow it with
 * cct_sgd_step(..., lambda = 0). */
int cct_l1_update(cct_ctx* ctx, size_t count, float* g, float lambda, const float* w);

#ifdef __cplusplus
}
#endif
#endif /* CCT_B200_H */
