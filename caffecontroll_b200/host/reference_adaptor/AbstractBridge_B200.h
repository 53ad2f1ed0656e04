// AbstractBridge for B200Driver.  The primary template's constructor asserts "change this for new devices"
// (src/bridges/AbstractBridge.h:132-156); this specialisation follows the reference's GPUDriver one (:445-631): the four
// cubes the bridge works on do not own memory, they are re-pointed at the layers' device cubes in every pass.
#ifndef _ABSTRACT_BRIDGE_B200_H
#define _ABSTRACT_BRIDGE_B200_H

#include "bridges/AbstractBridge.h"
#include "DeviceDriver_B200.h"

template <typename InputLayerDataType, LayoutType InputLayerLayout, typename OutputLayerDataType, LayoutType OutputLayerLayout>
class AbstractBridge<InputLayerDataType, InputLayerLayout, OutputLayerDataType, OutputLayerLayout, B200Driver> : public PhysicalOperator {
  public:
    typedef LogicalCube<InputLayerDataType, InputLayerLayout> InputCube;
    typedef LogicalCube<OutputLayerDataType, OutputLayerLayout> OutputCube;

  protected:
    size_t curr_B;
    // views (no memory of their own) of the layers' device cubes, re-pointed in every pass
    InputCube * input_d_cube, * input_g_cube;
    OutputCube * output_d_cube, * output_g_cube;

  public:
    std::string name;

    typedef Layer<InputLayerDataType, InputLayerLayout> InputLayerType;
    typedef Layer<OutputLayerDataType, OutputLayerLayout> OutputLayerType;

    const size_t iR, iC, iD, iB;
    const size_t oR, oC, oD, oB;

    InputLayerType * const p_input_layer;
    OutputLayerType * const p_output_layer;

    const cnn::LayerParameter * const layer_param;
    const cnn::SolverParameter * const solver_param;

    B200Driver * const p_driver;

    bool needs_to_calc_backward_grad;

    Report report_constructor;
    Report report_last_lowering;
    Report report_history;

    bool bias_term;

    virtual void set_model_cube(LogicalCube<InputLayerDataType, InputLayerLayout> * model) {}
    virtual LogicalCube<InputLayerDataType, InputLayerLayout> * const get_model_cube() { return NULL; }
    virtual void set_bias_cube(LogicalCube<InputLayerDataType, InputLayerLayout> * bias) {}
    virtual LogicalCube<InputLayerDataType, InputLayerLayout> * const get_bias_cube() { return NULL; }
    virtual LogicalCube<InputLayerDataType, InputLayerLayout> * const get_model_grad_cube() { return NULL; }
    LogicalCube<InputLayerDataType, InputLayerLayout> * const get_bias_grad_cube() { return NULL; }
    virtual GradientUpdater<InputLayerDataType, B200Driver> * const get_model_updater() { return NULL; }
    virtual GradientUpdater<InputLayerDataType, B200Driver> * const get_bias_updater() { return NULL; }

    void set_curr_batch_size(const size_t _curr_B) { curr_B = _curr_B; }

    AbstractBridge(InputLayerType * const _p_input_layer, OutputLayerType * const _p_output_layer,
        const cnn::LayerParameter * const _layer_param, const cnn::SolverParameter * const _solver_param,
        B200Driver * const _p_driver) :
      curr_B(_p_input_layer->p_data_cube->B), iR(_p_input_layer->p_data_cube->R), iC(_p_input_layer->p_data_cube->C),
      iD(_p_input_layer->p_data_cube->D), iB(_p_input_layer->p_data_cube->B), oR(_p_output_layer->p_data_cube->R),
      oC(_p_output_layer->p_data_cube->C), oD(_p_output_layer->p_data_cube->D), oB(_p_output_layer->p_data_cube->B),
      p_input_layer(_p_input_layer), p_output_layer(_p_output_layer), layer_param(_layer_param),
      solver_param(_solver_param), p_driver(_p_driver), needs_to_calc_backward_grad(true), bias_term(false) {
      input_d_cube = new LogicalCube<InputLayerDataType, InputLayerLayout>(NULL, iR, iC, iD, iB, p_driver);
      input_g_cube = new LogicalCube<InputLayerDataType, InputLayerLayout>(NULL, iR, iC, iD, iB, p_driver);
      output_d_cube = new LogicalCube<OutputLayerDataType, OutputLayerLayout>(NULL, oR, oC, oD, oB, p_driver);
      output_g_cube = new LogicalCube<OutputLayerDataType, OutputLayerLayout>(NULL, oR, oC, oD, oB, p_driver);
    }

    virtual ~AbstractBridge() {
      delete input_d_cube; delete input_g_cube; delete output_d_cube; delete output_g_cube;
    }

    virtual size_t get_input_data_size() { return input_d_cube->n_elements; }
    virtual size_t get_output_data_size() { return output_d_cube->n_elements; }
};

#endif
