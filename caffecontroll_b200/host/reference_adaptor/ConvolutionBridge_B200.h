// ConvolutionBridge for B200Driver: the specialisation a maintainer adds beside the CPU / GPU branches of
// src/bridges/ConvolutionBridge_impl.hxx (:294-500 forward, :551-773 backward).  Same public members as the reference's
// class (src/bridges/ConvolutionBridge.h:74-214); forward() and backward() are ONE C-ABI call each instead of the
// per-image lower / sgemm / bias loops.  All cubes are device cubes allocated through the driver.
#ifndef _CONVOLUTION_BRIDGE_B200_H
#define _CONVOLUTION_BRIDGE_B200_H

#include "bridges/ConvolutionBridge.h"
#include "AbstractBridge_B200.h"

template <>
class ConvolutionBridge<float, Layout_CRDB, float, Layout_CRDB, B200Driver>
: public AbstractBridge<float, Layout_CRDB, float, Layout_CRDB, B200Driver> {
  public:
    typedef AbstractBridge<float, Layout_CRDB, float, Layout_CRDB, B200Driver> Base;
    typedef Layer<float, Layout_CRDB> InputLayerType;
    typedef Layer<float, Layout_CRDB> OutputLayerType;
    typedef LogicalCube<float, Layout_CRDB> LogicalCubeType;

    const size_t K;
    const size_t num_output_features;
    const size_t stride;
    const size_t padding;
    const size_t group;   // cnn::ConvolutionParameter::group, honoured here (the reference bridge ignores it: src/DeepNet.h:1075-1077)

    const cnn::FillerParameter weight_filler;
    const cnn::FillerParameter bias_filler;

    LogicalCubeType * p_model_cube;   // points at the shadow, as in the reference
    LogicalCubeType * p_bias_cube;

    // The pbridge may hand the bridge its own (device) model / bias storage.
    void set_model_cube(LogicalCubeType * model) { p_model_cube_shadow->set_p_data(model->get_p_data()); }
    LogicalCubeType * const get_model_cube() { return p_model_cube_shadow; }
    void set_bias_cube(LogicalCubeType * bias) { if (p_bias_cube) p_bias_cube->set_p_data(bias->get_p_data()); }
    LogicalCubeType * const get_bias_cube() { return p_bias_cube; }
    LogicalCubeType * const get_model_grad_cube() { return p_model_gradient_cube; }
    LogicalCubeType * const get_bias_grad_cube() { return p_bias_gradient_cube; }

    ConvolutionBridge(InputLayerType * const _p_input_layer, OutputLayerType * const _p_output_layer,
        const cnn::LayerParameter * const _layer_param, const cnn::SolverParameter * const _solver_param,
        B200Driver * const _p_driver)
    : Base(_p_input_layer, _p_output_layer, _layer_param, _solver_param, _p_driver),
      K(layer_param->convolution_param().kernel_size()), num_output_features(layer_param->convolution_param().num_output()),
      stride(layer_param->convolution_param().stride()), padding(layer_param->convolution_param().pad()),
      group(layer_param->convolution_param().group()),
      weight_filler(layer_param->convolution_param().weight_filler()), bias_filler(layer_param->convolution_param().bias_filler()),
      p_model_cube(NULL), p_bias_cube(NULL), p_model_gradient_cube(NULL), p_model_cube_shadow(NULL),
      p_bias_gradient_cube(NULL), plan_(NULL) {
      report_forward_constructor.reset();
      bias_term = layer_param->convolution_param().bias_term();
      cct_conv_desc d = {(int) iB, (int) iD, (int) iR, (int) oD, (int) K, (int) stride, (int) padding, (int) group,
                         bias_term ? 1 : 0, CCT_ALGO_AUTO};
      int m = 0;
      p_driver->check(cct_conv_out_size(&d, &m), "cct_conv_out_size");
      assert(iR == iC && (size_t) m == oR && oR == oC && iB == oB && oD == num_output_features);
      p_driver->check(cct_conv_plan_create(p_driver->ctx(), &d, &plan_), "cct_conv_plan_create");
      p_model_cube_shadow = new LogicalCubeType(K, K, iD / group, oD, p_driver);
      initialize_logical_cube(p_model_cube_shadow, weight_filler);
      p_model_cube = new LogicalCubeType(p_model_cube_shadow->get_p_data(), K, K, iD / group, oD, p_driver);
      p_model_gradient_cube = new LogicalCubeType(K, K, iD / group, oD, p_driver);
      if (bias_term) {
        p_bias_cube = new LogicalCubeType(1, 1, oD, 1, p_driver);
        initialize_logical_cube(p_bias_cube, bias_filler);
        p_bias_gradient_cube = new LogicalCubeType(1, 1, oD, 1, p_driver);
      }
      report_forward_constructor.end(0, 0, 0);
    }

    ~ConvolutionBridge() {
      if (plan_) cct_conv_plan_destroy(plan_);
      delete p_model_cube; delete p_model_cube_shadow; delete p_model_gradient_cube;
      delete p_bias_cube; delete p_bias_gradient_cube;
    }

    void forward() {
      report_forward_last_transfer.reset();
      p_driver->check(cct_conv_forward(plan_, p_input_layer->p_data_cube->get_p_data(), p_model_cube_shadow->get_p_data(),
                                       bias_term ? p_bias_cube->get_p_data() : NULL, p_output_layer->p_data_cube->get_p_data(), 0),
                      "cct_conv_forward");
      // flops of the one GEMM, bytes read / written once (what the reference's Report of this bridge counts)
      report_forward_last_transfer.end(sizeof(float) * (p_input_layer->p_data_cube->n_elements + p_model_cube_shadow->n_elements),
                                       sizeof(float) * p_output_layer->p_data_cube->n_elements,
                                       2.0 * oD * (K * K * iD / group) * oR * oC * iB);
      report_forward_history.aggregate(report_forward_last_transfer);
    }

    // dW and db are overwritten, dX is written iff needs_to_calc_backward_grad, the output gradient is left untouched.
    void backward() {
      report_backward_updateweight_last_transfer.reset();
      p_driver->check(cct_conv_backward(plan_, p_input_layer->p_data_cube->get_p_data(), p_model_cube_shadow->get_p_data(),
                                        p_output_layer->p_gradient_cube->get_p_data(),
                                        needs_to_calc_backward_grad ? p_input_layer->p_gradient_cube->get_p_data() : NULL,
                                        p_model_gradient_cube->get_p_data(), bias_term ? p_bias_gradient_cube->get_p_data() : NULL),
                      "cct_conv_backward");
      const double gemm = 2.0 * oD * (K * K * iD / group) * oR * oC * iB;
      report_backward_updateweight_last_transfer.end(
          sizeof(float) * (p_output_layer->p_gradient_cube->n_elements + p_input_layer->p_data_cube->n_elements + p_model_cube_shadow->n_elements),
          sizeof(float) * (p_model_gradient_cube->n_elements + (needs_to_calc_backward_grad ? p_input_layer->p_gradient_cube->n_elements : 0)),
          (needs_to_calc_backward_grad ? 2.0 : 1.0) * gemm);
      report_backward_updateweight_history.aggregate(report_backward_updateweight_last_transfer);
    }

  protected:
    LogicalCubeType * p_model_gradient_cube;
    LogicalCubeType * p_model_cube_shadow;
    LogicalCubeType * p_bias_gradient_cube;
    cct_conv_plan * plan_;

    // src/bridges/ConvolutionBridge_impl.hxx:250-267
    void initialize_logical_cube(const LogicalCubeType * cube, const cnn::FillerParameter filler_param) {
      const std::string type = filler_param.type();
      DeviceMemoryPointer * data = cube->get_device_pointer(p_driver);
      if (type == "constant") p_driver->sconstant_initialize(data, filler_param.value());
      else if (type == "xavier") p_driver->sinitialize_xavier(data, cube->B, solver_param->random_seed());
      else if (type == "bernoulli") p_driver->sbernoulli_initialize(data, filler_param.value(), solver_param->random_seed());
      else if (type == "gaussian") p_driver->sgaussian_initialize(data, filler_param.mean(), filler_param.std(), solver_param->random_seed());
      else { std::cout << "ERROR! INITIALIZATION TYPE NOT SUPPORTED!" << std::endl; assert(false); }
    }
};

#endif
