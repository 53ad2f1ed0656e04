// Test infrastructure (oracle build only): plain structs standing in for the protoc-generated message
// classes of the reference's cnn.proto, so its bridges compile without protobuf.  Only the accessors the
// convolution / pooling / ReLU bridges, the parallelized bridge and the SGD updater read are present;
// defaults are the protobuf defaults of the schema (stride 1, pad 0, group 1, bias_term true,
// lr_policy "fixed" is never relied on: the wrapper always sets the solver fields it uses).
#ifndef CCT_ORACLE_SHIM_CNN_PB_H
#define CCT_ORACLE_SHIM_CNN_PB_H
#include <string>
#include <vector>
namespace cnn {

struct FillerParameter {
  std::string type_ = "constant";
  float value_ = 0.f, mean_ = 0.f, std_ = 1.f;
  const std::string& type() const { return type_; }
  float value() const { return value_; }
  float mean() const { return mean_; }
  float std() const { return std_; }
};

struct ConvolutionParameter {
  unsigned num_output_ = 0, kernel_size_ = 0, pad_ = 0, stride_ = 1, group_ = 1;
  bool bias_term_ = true;
  FillerParameter weight_filler_, bias_filler_;
  unsigned num_output() const { return num_output_; }
  unsigned kernel_size() const { return kernel_size_; }
  unsigned pad() const { return pad_; }
  unsigned stride() const { return stride_; }
  unsigned group() const { return group_; }
  bool bias_term() const { return bias_term_; }
  const FillerParameter& weight_filler() const { return weight_filler_; }
  const FillerParameter& bias_filler() const { return bias_filler_; }
};

struct PoolingParameter {
  unsigned kernel_size_ = 0, stride_ = 1;
  int pool_ = 0;
  unsigned kernel_size() const { return kernel_size_; }
  unsigned stride() const { return stride_; }
  int pool() const { return pool_; }
};

struct LRNParameter {
  unsigned local_size_ = 5;
  float alpha_ = 1.f, beta_ = 0.75f;
  unsigned local_size() const { return local_size_; }
  float alpha() const { return alpha_; }
  float beta() const { return beta_; }
};

struct DropoutParameter {
  float ratio_ = 0.5f;
  float dropout_ratio() const { return ratio_; }
};

struct InnerProductParameter {
  unsigned num_output_ = 0;
  bool bias_term_ = true;
  FillerParameter weight_filler_, bias_filler_;
  unsigned num_output() const { return num_output_; }
  bool bias_term() const { return bias_term_; }
  const FillerParameter& weight_filler() const { return weight_filler_; }
  const FillerParameter& bias_filler() const { return bias_filler_; }
};

struct ParamSpec {
  float lr_mult_ = 1.f, decay_mult_ = 1.f;
  float lr_mult() const { return lr_mult_; }
  float decay_mult() const { return decay_mult_; }
};

struct LayerParameter {
  ConvolutionParameter conv_;
  PoolingParameter pool_;
  LRNParameter lrn_;
  DropoutParameter dropout_;
  InnerProductParameter ip_;
  float gpu_batch_[4] = {0.f, 0.f, 0.f, 0.f};
  std::vector<float> blobs_lr_, weight_decay_;
  std::vector<ParamSpec> param_;
  const ConvolutionParameter& convolution_param() const { return conv_; }
  const PoolingParameter& pooling_param() const { return pool_; }
  const LRNParameter& lrn_param() const { return lrn_; }
  const DropoutParameter& dropout_param() const { return dropout_; }
  const InnerProductParameter& inner_product_param() const { return ip_; }
  float gpu_0_batch_proportion() const { return gpu_batch_[0]; }
  float gpu_1_batch_proportion() const { return gpu_batch_[1]; }
  float gpu_2_batch_proportion() const { return gpu_batch_[2]; }
  float gpu_3_batch_proportion() const { return gpu_batch_[3]; }
  int blobs_lr_size() const { return (int)blobs_lr_.size(); }
  float blobs_lr(int i) const { return blobs_lr_[i]; }
  int weight_decay_size() const { return (int)weight_decay_.size(); }
  float weight_decay(int i) const { return weight_decay_[i]; }
  int param_size() const { return (int)param_.size(); }
  const ParamSpec& param(int i) const { return param_[i]; }
};

struct SolverParameter {
  long random_seed_ = -1;
  std::string lr_policy_ = "fixed", regularization_type_ = "L2";
  float base_lr_ = 0.01f, gamma_ = 0.f, power_ = 0.f, momentum_ = 0.f, weight_decay_ = 0.f, delta_ = 1e-8f;
  int stepsize_ = 1, max_iter_ = 1;
  long random_seed() const { return random_seed_; }
  const std::string& lr_policy() const { return lr_policy_; }
  const std::string& regularization_type() const { return regularization_type_; }
  float base_lr() const { return base_lr_; }
  float gamma() const { return gamma_; }
  float power() const { return power_; }
  float momentum() const { return momentum_; }
  float weight_decay() const { return weight_decay_; }
  float delta() const { return delta_; }
  int stepsize() const { return stepsize_; }
  int max_iter() const { return max_iter_; }
};

}  // namespace cnn
#endif
