// Runs one convolution layer through the C++ bridge mirror (cct_host.h): forward, backward, and optionally the
// ParallelizedBridge's SGD step.  Inputs and outputs are raw fp32 files in a directory, so a test harness can feed the
// same tensors to a CPU checker:
//   host_selftest <dir> B D n o k s p g steps
// reads  X.bin W.bin b.bin dY.bin ; writes Y.bin dX.bin dW.bin db.bin Wnew.bin bnew.bin
#include <fstream>
#include <iostream>

#include "cct_host.h"

static std::vector<float> load(const std::string& path, size_t count) {
  std::vector<float> v(count);
  std::ifstream f(path, std::ios::binary);
  f.read(reinterpret_cast<char*>(v.data()), count * sizeof(float));
  if (!f) { std::cerr << "cannot read " << path << std::endl; std::exit(2); }
  return v;
}
static void save(const std::string& path, const std::vector<float>& v) {
  std::ofstream f(path, std::ios::binary);
  f.write(reinterpret_cast<const char*>(v.data()), v.size() * sizeof(float));
}

int main(int argc, char** argv) {
  if (argc < 11) { std::cerr << "usage: host_selftest dir B D n o k s p g steps [fc]" << std::endl; return 2; }
  const std::string dir = argv[1];
  const int B = atoi(argv[2]), D = atoi(argv[3]), n = atoi(argv[4]), o = atoi(argv[5]), k = atoi(argv[6]), s = atoi(argv[7]),
            p = atoi(argv[8]), g = atoi(argv[9]), steps = atoi(argv[10]);
  const int m = (n + 2 * p - k) / s + 1;
  using namespace cct;
  B200Driver driver(0);
  LogicalCube<float> x(n, n, D, B, &driver), dx(n, n, D, B, &driver), y(m, m, o, B, &driver), dy(m, m, o, B, &driver);
  Layer in(&x, &dx), out(&y, &dy);
  ConvolutionParameter cp;
  cp.num_output = o; cp.kernel_size = k; cp.stride = s; cp.pad = p; cp.group = g; cp.bias_term = true;
  ConvolutionBridge conv(&in, &out, cp, &driver);
  SolverParameter solver;  // lr 0.01 "step", momentum 0.9, decay 0.0005
  ParallelizedBridge pbridge(&conv, &solver, &driver);
  x.copy_from_host(load(dir + "/X.bin", x.n_elements).data());
  dy.copy_from_host(load(dir + "/dY.bin", dy.n_elements).data());
  conv.get_model_cube()->copy_from_host(load(dir + "/W.bin", conv.get_model_cube()->n_elements).data());
  conv.get_bias_cube()->copy_from_host(load(dir + "/b.bin", o).data());

  pbridge.set_update_model_gradients(false);
  pbridge.forward();
  pbridge.backward();
  driver.device_sync();
  std::vector<float> hy(y.n_elements), hdx(dx.n_elements), hdw(conv.get_model_cube()->n_elements), hdb(o);
  y.copy_to_host(hy.data()); dx.copy_to_host(hdx.data());
  conv.get_model_grad_cube()->copy_to_host(hdw.data()); conv.get_bias_grad_cube()->copy_to_host(hdb.data());
  save(dir + "/Y.bin", hy); save(dir + "/dX.bin", hdx); save(dir + "/dW.bin", hdw); save(dir + "/db.bin", hdb);

  pbridge.set_update_model_gradients(true);
  for (int i = 0; i < steps; ++i) { pbridge.forward(); pbridge.backward(); }
  driver.device_sync();
  std::vector<float> hw(hdw.size()), hb(o);
  conv.get_model_cube()->copy_to_host(hw.data()); conv.get_bias_cube()->copy_to_host(hb.data());
  save(dir + "/Wnew.bin", hw); save(dir + "/bnew.bin", hb);
  if (argc > 11 && std::string(argv[11]) == "fc") {
    // kernel == input: the same layer through FullyConnectedBridge (a 1x1 convolution over the flattened input)
    FullyConnectedBridge fc(&in, &out, o, true, &driver);
    ConvolutionBridge& c = fc.as_convolution();
    c.get_model_cube()->copy_from_host(load(dir + "/W.bin", c.get_model_cube()->n_elements).data());
    c.get_bias_cube()->copy_from_host(load(dir + "/b.bin", o).data());
    fc.forward();
    fc.backward();
    driver.device_sync();
    y.copy_to_host(hy.data()); dx.copy_to_host(hdx.data());
    c.get_model_grad_cube()->copy_to_host(hdw.data()); c.get_bias_grad_cube()->copy_to_host(hdb.data());
    save(dir + "/Y_fc.bin", hy); save(dir + "/dX_fc.bin", hdx); save(dir + "/dW_fc.bin", hdw); save(dir + "/db_fc.bin", hdb);
  }
  std::cout << "host_selftest ok" << std::endl;
  return 0;
}
