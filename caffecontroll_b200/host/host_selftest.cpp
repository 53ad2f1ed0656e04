// Runs one convolution layer through the C++ bridge mirror (cct_host.h): forward, backward, and optionally the
// ParallelizedBridge's SGD step.  Inputs and outputs are raw fp32 files in a directory, so a test harness can feed the
// same tensors to a CPU checker:
//   host_selftest <dir> B D n o k s p g steps [fc | ranks=N]
// reads  X.bin W.bin b.bin dY.bin ; writes Y.bin dX.bin dW.bin db.bin Wnew.bin bnew.bin
//   fc       additionally runs the same tensors through FullyConnectedBridge (needs k == n: an inner product)
//   ranks=N  additionally splits the batch over N GPUs, one host thread and one B200Driver per GPU (as the reference's
//            PhysicalStratum runs its partitions), gradients summed by the C ABI's NCCL communicator; writes
//            Wnew_r<rank>.bin / bnew_r<rank>.bin after `steps` updates - every rank must hold the single-GPU result
#include <thread>
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
  const std::string mode = argc > 11 ? argv[11] : "";
  if (mode == "fc") {
    // kernel == input: the same layer through FullyConnectedBridge (tensor-core GEMMs over the flattened input)
    FullyConnectedBridge fc(&in, &out, o, true, &driver);
    fc.get_model_cube()->copy_from_host(load(dir + "/W.bin", fc.get_model_cube()->n_elements).data());
    fc.get_bias_cube()->copy_from_host(load(dir + "/b.bin", o).data());
    fc.forward();
    fc.backward();
    driver.device_sync();
    y.copy_to_host(hy.data()); dx.copy_to_host(hdx.data());
    fc.get_model_grad_cube()->copy_to_host(hdw.data()); fc.get_bias_grad_cube()->copy_to_host(hdb.data());
    save(dir + "/Y_fc.bin", hy); save(dir + "/dX_fc.bin", hdx); save(dir + "/dW_fc.bin", hdw); save(dir + "/db_fc.bin", hdb);
  }
  if (mode.compare(0, 6, "ranks=") == 0) {
    const int ranks = atoi(mode.c_str() + 6);
    if (ranks < 2 || B % ranks) { std::cerr << "ranks must be >= 2 and divide the batch" << std::endl; return 2; }
    const std::vector<unsigned char> id = Communicator::unique_id();
    const std::vector<float> hX = load(dir + "/X.bin", x.n_elements), hdY = load(dir + "/dY.bin", dy.n_elements),
                             hW = load(dir + "/W.bin", hdw.size()), hb0 = load(dir + "/b.bin", o);
    const int Bp = B / ranks;
    std::vector<std::thread> threads;
    for (int r = 0; r < ranks; ++r)
      threads.emplace_back([&, r]() {
        B200Driver drv(r);
        Communicator comm(&drv, ranks, r, id.data());
        LogicalCube<float> px(n, n, D, Bp, &drv), pdx(n, n, D, Bp, &drv), py(m, m, o, Bp, &drv), pdy(m, m, o, Bp, &drv);
        Layer pin(&px, &pdx), pout(&py, &pdy);
        ConvolutionBridge sub(&pin, &pout, cp, &drv);
        ParallelizedBridge pb(&sub, &solver, &drv, &comm);
        px.copy_from_host(hX.data() + (size_t)r * px.n_elements);    // contiguous batch slices, partition r
        pdy.copy_from_host(hdY.data() + (size_t)r * pdy.n_elements);
        sub.get_model_cube()->copy_from_host(hW.data());
        sub.get_bias_cube()->copy_from_host(hb0.data());
        for (int i = 0; i < steps; ++i) { pb.forward(); pb.backward(); }
        drv.device_sync();
        std::vector<float> w(hW.size()), b(o);
        sub.get_model_cube()->copy_to_host(w.data()); sub.get_bias_cube()->copy_to_host(b.data());
        save(dir + "/Wnew_r" + std::to_string(r) + ".bin", w); save(dir + "/bnew_r" + std::to_string(r) + ".bin", b);
      });
    for (auto& t : threads) t.join();
  }
  if (mode.compare(0, 5, "mpfc=") == 0) {
    // kernel == input: the layer as a fully connected one split over `ranks` GPUs by output depth, one host thread each
    const int ranks = atoi(mode.c_str() + 5);
    if (ranks < 2 || B % ranks || o % ranks) { std::cerr << "ranks must be >= 2 and divide batch and outputs" << std::endl; return 2; }
    const std::vector<unsigned char> id = Communicator::unique_id();
    const std::vector<float> hX = load(dir + "/X.bin", x.n_elements), hdY = load(dir + "/dY.bin", dy.n_elements),
                             hW = load(dir + "/W.bin", hdw.size()), hb0 = load(dir + "/b.bin", o);
    const int Bp = B / ranks, os = o / ranks;
    std::vector<std::thread> threads;
    for (int r = 0; r < ranks; ++r)
      threads.emplace_back([&, r]() {
        B200Driver drv(r);
        Communicator comm(&drv, ranks, r, id.data());
        LogicalCube<float> px(n, n, D, Bp, &drv), pdx(n, n, D, Bp, &drv), py(1, 1, o, Bp, &drv), pdy(1, 1, o, Bp, &drv);
        Layer pin(&px, &pdx), pout(&py, &pdy);
        ModelParallelFullyConnectedBridge sub(&pin, &pout, o, true, &drv, &comm);
        ParallelizedBridgeT<ModelParallelFullyConnectedBridge> pb(&sub, &solver, &drv, nullptr);  // slice gradients need no sum
        pb.set_update_model_gradients(false);
        px.copy_from_host(hX.data() + (size_t)r * px.n_elements);
        pdy.copy_from_host(hdY.data() + (size_t)r * pdy.n_elements);
        const size_t nw = sub.get_model_cube()->n_elements;  // rows r * os ... of the [o][D n n] matrix
        sub.get_model_cube()->copy_from_host(hW.data() + (size_t)r * nw);
        sub.get_bias_cube()->copy_from_host(hb0.data() + (size_t)r * os);
        pb.forward();
        pb.backward();
        drv.device_sync();
        std::vector<float> vy(py.n_elements), vdx(pdx.n_elements), vdw(nw), vdb(os);
        py.copy_to_host(vy.data()); pdx.copy_to_host(vdx.data());
        sub.get_model_grad_cube()->copy_to_host(vdw.data()); sub.get_bias_grad_cube()->copy_to_host(vdb.data());
        const std::string tag = "_mp" + std::to_string(r) + ".bin";
        save(dir + "/Y" + tag, vy); save(dir + "/dX" + tag, vdx); save(dir + "/dW" + tag, vdw); save(dir + "/db" + tag, vdb);
      });
    for (auto& t : threads) t.join();
  }
  std::cout << "host_selftest ok" << std::endl;
  return 0;
}
