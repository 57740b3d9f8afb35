// The smallest complete program: start the context from switchml.cfg, submit a few
// asynchronous allreduce jobs, wait, stop, check the sums.
// Counterpart of the reference's examples/hello_world/main.cc (8 float tensors of 2^15
// elements, out of place, result must be input x num_workers within 1 % and the input
// must be untouched). With backend = cuda the buffers are placed on the GPU.
#include <cmath>
#include <cstdio>
#include <vector>

#include <cuda_runtime.h>

#include "switchml/context.h"

int main() {
  switchml::Context& ctx = switchml::Context::GetInstance();
  printf("Hello world! Starting the switchml context\n");
  if (!ctx.Start()) {
    fprintf(stderr, "could not start: is there a switchml.cfg in this directory?\n");
    return 1;
  }
  const uint64_t numel = 1 << 15;
  const int num_tensors = 8;
  const int num_workers = ctx.GetConfig().general_.num_workers;
  const bool on_gpu = ctx.GetConfig().general_.backend == "cuda";

  std::vector<std::vector<float>> in(num_tensors, std::vector<float>(numel)), out = in;
  for (int i = 0; i < num_tensors; i++)
    for (uint64_t j = 0; j < numel; j++) in[i][j] = static_cast<float>(i * numel + j);

  std::vector<float*> d_in(num_tensors, nullptr), d_out(num_tensors, nullptr);
  if (on_gpu) {
    for (int i = 0; i < num_tensors; i++) {
      cudaMalloc(&d_in[i], numel * 4);
      cudaMalloc(&d_out[i], numel * 4);
      cudaMemcpy(d_in[i], in[i].data(), numel * 4, cudaMemcpyHostToDevice);
    }
  }
  printf("Submitting all reduce jobs\n");
  for (int i = 0; i < num_tensors; i++) {
    float* src = on_gpu ? d_in[i] : in[i].data();
    float* dst = on_gpu ? d_out[i] : out[i].data();
    ctx.AllReduceAsync(src, dst, numel, switchml::FLOAT32, switchml::SUM);
  }
  printf("Waiting for all jobs to finish\n");
  ctx.WaitForAllJobs();
  std::vector<std::vector<float>> in_after = in;
  if (on_gpu) {
    for (int i = 0; i < num_tensors; i++) {
      cudaMemcpy(out[i].data(), d_out[i], numel * 4, cudaMemcpyDeviceToHost);
      cudaMemcpy(in_after[i].data(), d_in[i], numel * 4, cudaMemcpyDeviceToHost);
      cudaFree(d_in[i]);
      cudaFree(d_out[i]);
    }
  }
  printf("Stopping the switchml context\n");
  ctx.Stop();

  printf("Verifying results\n");
  for (int i = 0; i < num_tensors; i++) {
    for (uint64_t j = 0; j < numel; j++) {
      float expected = in[i][j] * num_workers;
      float err = std::fabs(expected - out[i][j]) / (std::fabs(expected) + 1e-6f) * 100.0f;
      if (err > 1.0f) {
        printf("Element %lu of tensor %d is %e, expected %e (error %.2f%%)\n",
               static_cast<unsigned long>(j), i, out[i][j], expected, err);
        return 1;
      }
      if (in_after[i][j] != in[i][j]) {
        printf("Input element %lu of tensor %d was modified\n", static_cast<unsigned long>(j), i);
        return 1;
      }
    }
  }
  printf("Data verified successfully, exiting\n");
  return 0;
}
