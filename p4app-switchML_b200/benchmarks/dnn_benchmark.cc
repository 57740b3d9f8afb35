// Training-loop model: how much of the gradient communication hides behind compute.
//
// Counterpart of the reference's benchmarks/dnn_benchmark/main.cc. A model is a CSV of
// layers "layer_index,numel,forward_pass_ns,backward_pass_ns" (models/*.csv). One
// iteration walks the layers forward — first waiting for that layer's pending allreduce,
// then sleeping its forward time — and backward in reverse order — sleeping the backward
// time, then launching that layer's allreduce asynchronously. Reports iterations/s.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <fstream>
#include <iostream>
#include <numeric>
#include <sstream>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "switchml/cli_flags.h"
#include "switchml/context.h"

struct Layer {
  uint64_t numel = 0, fwd_ns = 0, bwd_ns = 0;
  float* data = nullptr;
  std::shared_ptr<switchml::Job> job;
};

static bool LoadModel(const std::string& path, std::vector<Layer>* layers) {
  std::ifstream in(path);
  if (!in.good()) return false;
  std::string line;
  while (std::getline(in, line)) {
    if (line.empty() || !isdigit(static_cast<unsigned char>(line[0]))) continue;  // header / comments
    std::stringstream ss(line);
    std::string tok;
    std::vector<uint64_t> v;
    while (std::getline(ss, tok, ',')) v.push_back(strtoull(tok.c_str(), nullptr, 10));
    if (v.size() != 4) return false;
    Layer l;
    l.numel = v[1];
    l.fwd_ns = v[2];
    l.bwd_ns = v[3];
    layers->push_back(l);
  }
  return !layers->empty();
}

int main(int argc, char** argv) {
  switchml::CliFlags f;
  f.Add("model", "models/example.csv", "CSV file describing the layers.")
      .Add("device", "cpu", "cpu or gpu (gpu needs backend = cuda).")
      .Add("num-iters", "10", "Timed training iterations.")
      .Add("num-warmup-iters", "5", "Untimed iterations first.")
      .Add("verify", "false", "Check that every layer ends up as input x n^iterations.");
  if (!f.Parse(argc, argv, "DNN communication benchmark")) return 1;
  std::vector<Layer> layers;
  if (!LoadModel(f.Str("model"), &layers)) {
    std::cerr << "cannot read model '" << f.Str("model") << "'" << std::endl;
    return 1;
  }
  const bool gpu = f.Str("device") == "gpu";
  const uint64_t iters = f.U64("num-iters"), warmup = f.U64("num-warmup-iters");
  switchml::Context& ctx = switchml::Context::GetInstance();
  if (!ctx.Start()) return 1;
  const int n = ctx.GetConfig().general_.num_workers;

  uint64_t total = 0;
  for (Layer& l : layers) {
    std::vector<float> init(l.numel, 1.0f);
    if (gpu) {
      cudaMalloc(&l.data, l.numel * 4);
      cudaMemcpy(l.data, init.data(), l.numel * 4, cudaMemcpyHostToDevice);
    } else {
      l.data = new float[l.numel];
      std::copy(init.begin(), init.end(), l.data);
    }
    total += l.numel;
  }
  std::cout << "Model with " << layers.size() << " layers, " << total << " parameters" << std::endl;

  std::vector<double> dur;
  auto begin = switchml::clock::now();
  for (uint64_t it = 0; it < iters + warmup; it++) {
    for (Layer& l : layers) {  // forward
      if (l.job) l.job->WaitToComplete();
      std::this_thread::sleep_for(std::chrono::nanoseconds(l.fwd_ns));
    }
    for (auto l = layers.rbegin(); l != layers.rend(); ++l) {  // backward
      std::this_thread::sleep_for(std::chrono::nanoseconds(l->bwd_ns));
      l->job = ctx.AllReduceAsync(l->data, l->data, l->numel, switchml::FLOAT32, switchml::SUM);
    }
    if (it >= warmup) {
      auto end = switchml::clock::now();
      dur.push_back(std::chrono::duration_cast<std::chrono::nanoseconds>(end - begin).count());
      begin = end;
      std::cout << "Iteration #" << it << "# finished. Duration: #" << dur.back() << "# ns Rate: #"
                << 1e9 / dur.back() << "# iter/s." << std::endl;
    } else {
      begin = switchml::clock::now();
    }
  }
  ctx.WaitForAllJobs();

  int rc = 0;
  if (f.Bool("verify")) {
    // Every worker started from ones, so after k sums each element is n^k. Values beyond
    // the float range would not verify: keep iterations x log2(n) below 127.
    double want = std::pow(static_cast<double>(n), static_cast<double>(iters + warmup));
    for (Layer& l : layers) {
      std::vector<float> got(l.numel);
      if (gpu) cudaMemcpy(got.data(), l.data, l.numel * 4, cudaMemcpyDeviceToHost);
      else std::copy(l.data, l.data + l.numel, got.begin());
      for (uint64_t i = 0; i < l.numel; i++) {
        if (std::fabs(got[i] - want) > std::fabs(want) * 0.01) {
          std::cout << "Verification failed: element " << i << " is " << got[i] << ", expected " << want << std::endl;
          rc = 1;
          break;
        }
      }
    }
    if (!rc) std::cout << "Results verified successfully." << std::endl;
  }
  std::sort(dur.begin(), dur.end());
  double mean = std::accumulate(dur.begin(), dur.end(), 0.0) / dur.size();
  std::cout << "Iterations/s min: #" << 1e9 / dur.back() << "# max: #" << 1e9 / dur.front() << "# median: #"
            << 1e9 / dur[dur.size() / 2] << "# mean: #" << 1e9 / mean << "#" << std::endl;
  ctx.Stop();
  for (Layer& l : layers) {
    if (gpu) cudaFree(l.data);
    else delete[] l.data;
  }
  return rc;
}
