// ParallelizedBridge_B200: what replaces ParallelizedBridge<DataType, BridgeType> (src/bridges/ParallelizedBridge.h:46-771,
// _impl.hxx) when a layer's mini-batch partition runs on a B200.  One process = one partition = one GPU; the batch slices
// of the other ranks live in other processes, and their model gradients are summed by an NCCL all-reduce
// (cct_allreduce_sum) in place of the reference's host-staged gather + serial sum (_impl.hxx:876-971).
//
// Towards DeepNet it is what the reference's pbridge is: an AbstractBridge<..., CPUDriver> whose input / output layers are
// HOST cubes, with the scheduler-facing virtuals of src/bridges/AbstractBridge.h:390-441 implemented (model / bias host
// copies on demand, gradient host copies, iteration counter, history copies), so model files and snapshots keep working.
// Inside: device cubes, the B200 sub-bridge, and the reference's own SGDGradientUpdater instantiated on B200Driver - the
// parameters, their gradients and the momentum history never leave the GPU.
#ifndef _PARALLELIZED_BRIDGE_B200_H
#define _PARALLELIZED_BRIDGE_B200_H

#include "bridges/AbstractBridge.h"
#include "ConvolutionBridge_B200.h"

template <typename DataType,
          template <typename, LayoutType, typename, LayoutType, typename> class BridgeType>
class ParallelizedBridge_B200 : public AbstractBridge<DataType, Layout_CRDB, DataType, Layout_CRDB, CPUDriver> {
  public:
    typedef AbstractBridge<DataType, Layout_CRDB, DataType, Layout_CRDB, CPUDriver> Base;
    typedef LogicalCube<DataType, Layout_CRDB> LogicalCubeType;
    typedef Layer<DataType, Layout_CRDB> LayerType;
    typedef BridgeType<DataType, Layout_CRDB, DataType, Layout_CRDB, B200Driver> SubBridge;

    using Base::p_input_layer; using Base::p_output_layer; using Base::needs_to_calc_backward_grad; using Base::bias_term;
    using Base::report_forward_last_transfer; using Base::report_forward_history;
    using Base::report_backward_updateweight_last_transfer; using Base::report_backward_updateweight_history;

    // `comm` sums gradients over the job's partitions (NULL: this is the only partition); it must belong to driver->ctx().
    ParallelizedBridge_B200(LayerType * const _input_layer, LayerType * const _output_layer,
        const cnn::LayerParameter * const _layer_param, const cnn::SolverParameter * const _solver_param,
        CPUDriver * const _p_cpu_driver, B200Driver * const _p_driver, cct_comm * _comm = NULL)
    : Base(_input_layer, _output_layer, _layer_param, _solver_param, _p_cpu_driver), driver(_p_driver), comm(_comm),
      update_model_gradients(true), model_host(NULL), bias_host(NULL), model_grad_host(NULL), bias_grad_host(NULL),
      updater(NULL), updater_bias(NULL) {
      const LogicalCubeType * x = _input_layer->p_data_cube, * y = _output_layer->p_data_cube;
      d_x = new LogicalCubeType(x->R, x->C, x->D, x->B, driver); d_dx = new LogicalCubeType(x->R, x->C, x->D, x->B, driver);
      d_y = new LogicalCubeType(y->R, y->C, y->D, y->B, driver); d_dy = new LogicalCubeType(y->R, y->C, y->D, y->B, driver);
      d_in = new LayerType(d_x, d_dx); d_out = new LayerType(d_y, d_dy);
      sub = new SubBridge(d_in, d_out, _layer_param, _solver_param, driver);
      bias_term = sub->bias_term;
      // per-blob multipliers: the old blobs_lr / weight_decay lists, then param { lr_mult decay_mult } (_impl.hxx:343-361, 429-447)
      float lr[2] = {1.f, 1.f}, reg[2] = {1.f, 1.f};
      for (int j = 0; j < 2; ++j) {
        if (_layer_param->blobs_lr_size() > j) lr[j] = _layer_param->blobs_lr(j);
        if (_layer_param->weight_decay_size() > j) reg[j] = _layer_param->weight_decay(j);
        if (_layer_param->param_size() > j) { lr[j] = _layer_param->param(j).lr_mult(); reg[j] = _layer_param->param(j).decay_mult(); }
      }
      LogicalCubeType * w = sub->get_model_cube();
      model_host = new LogicalCubeType(w->R, w->C, w->D, w->B);
      model_grad_host = new LogicalCubeType(w->R, w->C, w->D, w->B);
      updater = new SGDGradientUpdater<DataType, B200Driver>(w->n_elements, w->get_p_data(), _solver_param, lr[0], reg[0], driver);
      if (bias_term) {
        LogicalCubeType * b = sub->get_bias_cube();
        bias_host = new LogicalCubeType(b->R, b->C, b->D, b->B);
        bias_grad_host = new LogicalCubeType(b->R, b->C, b->D, b->B);
        updater_bias = new SGDGradientUpdater<DataType, B200Driver>(b->n_elements, b->get_p_data(), _solver_param, lr[1], reg[1], driver);
      }
      force_device_to_host_model_copy();
      if (bias_term) force_device_to_host_bias_copy();
    }

    ~ParallelizedBridge_B200() {
      delete updater; delete updater_bias; delete sub;
      delete d_in; delete d_out;  // a Layer deletes its cubes
      delete model_host; delete bias_host; delete model_grad_host; delete bias_grad_host;
    }

    // host input -> device, sub-bridge forward, device -> host output (src/bridges/ParallelizedBridge_impl.hxx:595-738)
    void forward() {
      report_forward_last_transfer.reset();
      copy(d_x, p_input_layer->p_data_cube, true);
      sub->forward();
      copy(p_output_layer->p_data_cube, d_y, false);
      report_forward_last_transfer.end();
      report_forward_history.aggregate(report_forward_last_transfer);
    }

    // host dY -> device, sub-bridge backward, gradient sum over the partitions, SGD on the device, dX -> host (:761-1141)
    void backward() {
      report_backward_updateweight_last_transfer.reset();
      sub->needs_to_calc_backward_grad = needs_to_calc_backward_grad;
      copy(d_dy, p_output_layer->p_gradient_cube, true);
      sub->backward();
      LogicalCubeType * gw = sub->get_model_grad_cube(), * gb = bias_term ? sub->get_bias_grad_cube() : NULL;
      if (comm) {
        driver->check(cct_allreduce_sum_begin(comm, gw->get_p_data(), gw->n_elements), "cct_allreduce_sum_begin");
        if (gb) driver->check(cct_allreduce_sum_begin(comm, gb->get_p_data(), gb->n_elements), "cct_allreduce_sum_begin");
        driver->check(cct_comm_wait(comm), "cct_comm_wait");
      }
      if (update_model_gradients) {
        updater->update(gw->get_p_data());
        if (gb) updater_bias->update(gb->get_p_data());
      }
      if (needs_to_calc_backward_grad) copy(p_input_layer->p_gradient_cube, d_dx, false);
      driver->device_sync();
      report_backward_updateweight_last_transfer.end();
      report_backward_updateweight_history.aggregate(report_backward_updateweight_last_transfer);
    }

    // ---- what DeepNet and the tests read (names as in src/bridges/ParallelizedBridge.h)
    LogicalCubeType * const get_model_cube() { force_device_to_host_model_copy(); return model_host; }
    LogicalCubeType * const get_bias_cube() { if (!bias_term) return NULL; force_device_to_host_bias_copy(); return bias_host; }
    void set_model_cube(LogicalCubeType * model) { copy(sub->get_model_cube(), model, true); }
    void set_bias_cube(LogicalCubeType * bias) { if (bias_term) copy(sub->get_bias_cube(), bias, true); }
    GradientUpdater<DataType, B200Driver> * get_device_model_updater() { return updater; }

    // ---- scheduler-facing virtuals (src/bridges/AbstractBridge.h:390-441)
    void set_share_pointer_with_prev_bridge(bool) {}
    bool get_share_pointer_with_prev_bridge() { return false; }
    void set_share_pointer_with_next_bridge(bool) {}
    bool get_share_pointer_with_next_bridge() { return false; }
    size_t get_num_partitions_CPU() { return 0; }
    std::vector<size_t> get_GPU_batch_sizes() { return std::vector<size_t>(1, p_input_layer->p_data_cube->B); }
    std::vector<int> get_used_gpu_to_device_id_map() { return std::vector<int>(1, driver->gpu_id); }
    std::vector<LogicalCubeType *> get_data_cubes_higher() { return std::vector<LogicalCubeType *>(1, d_y); }
    std::vector<LogicalCubeType *> get_grad_cubes_higher() { return std::vector<LogicalCubeType *>(1, d_dy); }
    void force_host_to_device_model_copy() { copy(sub->get_model_cube(), model_host, true); }
    void force_host_to_device_bias_copy() { if (bias_term) copy(sub->get_bias_cube(), bias_host, true); }
    void force_device_to_host_model_copy() { copy(model_host, sub->get_model_cube(), false); }
    void force_device_to_host_bias_copy() { if (bias_term) copy(bias_host, sub->get_bias_cube(), false); }
    DataType * get_model_gradient_host() { copy(model_grad_host, sub->get_model_grad_cube(), false); return model_grad_host->get_p_data(); }
    DataType * get_bias_gradient_host() {
      if (!bias_term) return NULL;
      copy(bias_grad_host, sub->get_bias_grad_cube(), false);
      return bias_grad_host->get_p_data();
    }
    void update_model_with_gradient_CPU(DataType * grad) {  // a gradient computed elsewhere: upload it, step on the device
      LogicalCubeType tmp(grad, model_grad_host->R, model_grad_host->C, model_grad_host->D, model_grad_host->B);
      copy(sub->get_model_grad_cube(), &tmp, true);
      updater->update(sub->get_model_grad_cube()->get_p_data());
    }
    void update_bias_with_gradient_CPU(DataType * grad) {
      if (!bias_term) return;
      LogicalCubeType tmp(grad, bias_grad_host->R, bias_grad_host->C, bias_grad_host->D, bias_grad_host->B);
      copy(sub->get_bias_grad_cube(), &tmp, true);
      updater_bias->update(sub->get_bias_grad_cube()->get_p_data());
    }
    void set_update_model_gradients(bool v) { update_model_gradients = v; }
    void set_current_iter(int it) { updater->set_current_iter(it); if (updater_bias) updater_bias->set_current_iter(it); }
    void force_device_to_host_model_history_copy() { updater->force_device_to_host_history_copy(); }
    void force_host_to_device_model_history_copy() { updater->force_host_to_device_history_copy(); }
    void force_device_to_host_bias_history_copy() { if (updater_bias) updater_bias->force_device_to_host_history_copy(); }
    void force_host_to_device_bias_history_copy() { if (updater_bias) updater_bias->force_host_to_device_history_copy(); }
    DataType * get_model_history_host_ptr() { return updater->get_p_history_updates_cube()->get_p_data(); }
    DataType * get_bias_history_host_ptr() { return updater_bias ? updater_bias->get_p_history_updates_cube()->get_p_data() : NULL; }
    void set_model_parallelism_group_size(int g) { assert(g == 1); }

    SubBridge * sub;

  private:
    B200Driver * const driver;
    cct_comm * const comm;
    bool update_model_gradients;
    LogicalCubeType * d_x, * d_dx, * d_y, * d_dy;
    LayerType * d_in, * d_out;
    LogicalCubeType * model_host, * bias_host, * model_grad_host, * bias_grad_host;
    SGDGradientUpdater<DataType, B200Driver> * updater, * updater_bias;

    // one of the two cubes is a host cube (CPUDriver's pointers are DEVICEMEMORY_LOCAL_RAM), the other lives on the GPU
    void copy(LogicalCubeType * dst, LogicalCubeType * src, bool to_device) {
      CPUDriver * host = Base::p_driver;
      if (to_device) driver->memcpy(dst->get_device_pointer(driver), src->get_device_pointer(host));
      else driver->memcpy(dst->get_device_pointer(host), src->get_device_pointer(driver));
    }
};

#endif
