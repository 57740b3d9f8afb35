// Allreduce benchmark straight on the C++ API.
//
// Counterpart of the reference's benchmarks/allreduce_benchmark/main.cc: same options
// (--tensor-numel 2^28, --tensor-type int32|float, --device cpu|gpu, --num-jobs 10,
// --num-warmup-jobs 5, --inplace, --verify, --sync-every, --err, --random, --seed,
// --dump-stats), same "#value#" output lines for scraping, goodput = numel*32 bit / ns,
// min/max/median/mean/stdev at the end, Ctrl-C stops the context cleanly. Differences:
// the verification takes the absolute error and uses bounded values, and with
// --device gpu the jobs are real GPU jobs (the reference can only allocate GPU buffers,
// no backend of its own accepts them).
#include <signal.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <numeric>
#include <random>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "switchml/cli_flags.h"
#include "switchml/context.h"

static std::atomic<bool> g_stop{false};

static void SignalThread(sigset_t set) {
  int sig = 0;
  sigwait(&set, &sig);
  g_stop = true;
  std::cout << "Signal " << sig << " received: stopping the context" << std::endl;
  switchml::Context& ctx = switchml::Context::GetInstance();
  if (ctx.GetContextState() == switchml::Context::RUNNING) ctx.Stop();
  exit(EXIT_SUCCESS);
}

template <typename T>
static void Describe(const char* what, std::vector<T> v, const char* unit) {
  if (v.empty()) return;
  std::sort(v.begin(), v.end());
  double sum = std::accumulate(v.begin(), v.end(), 0.0), mean = sum / v.size(), var = 0;
  for (T x : v) var += (x - mean) * (x - mean);
  std::cout << what << " min: #" << v.front() << "# max: #" << v.back() << "# median: #" << v[v.size() / 2]
            << "# mean: #" << mean << "# stdev: #" << std::sqrt(var / v.size()) << "# " << unit << std::endl;
}

int main(int argc, char** argv) {
  switchml::CliFlags f;
  f.Add("tensor-numel", "268435456", "Number of elements to all reduce.")
      .Add("tensor-type", "int32", "Data type: float or int32.")
      .Add("device", "cpu", "Where the tensors live: cpu or gpu (gpu needs backend = cuda).")
      .Add("num-jobs", "10", "Timed allreduce jobs.")
      .Add("num-warmup-jobs", "5", "Untimed jobs before the timed ones.")
      .Add("inplace", "true", "Use the same buffer as source and destination.")
      .Add("verify", "false", "Check the results.")
      .Add("sync-every", "1", "Wait for the submitted jobs after this many (0 = only at the end).")
      .Add("err", "1", "Allowed error in percent when verifying float results.")
      .Add("random", "false", "Initialise with random values instead of the +-i pattern.")
      .Add("seed", "0", "Seed of the random generator (0 = from the clock).")
      .Add("dump-stats", "false", "Print and clear the statistics after each sync.");
  if (!f.Parse(argc, argv, "Allreduce benchmark")) return 1;
  const uint64_t numel = f.U64("tensor-numel");
  const bool is_float = f.Str("tensor-type") == "float";
  const bool gpu = f.Str("device") == "gpu";
  const uint32_t num_jobs = f.U64("num-jobs"), num_warmup = f.U64("num-warmup-jobs");
  const bool inplace = f.Bool("inplace"), verify = f.Bool("verify");
  uint32_t sync_every = f.U64("sync-every");
  if (sync_every == 0) sync_every = num_jobs;

  sigset_t set;
  sigemptyset(&set);
  sigaddset(&set, SIGINT);
  sigaddset(&set, SIGTERM);
  pthread_sigmask(SIG_BLOCK, &set, nullptr);
  std::thread(SignalThread, set).detach();

  switchml::Context& ctx = switchml::Context::GetInstance();
  if (!ctx.Start()) return 1;
  const int n = ctx.GetConfig().general_.num_workers;
  if (gpu && ctx.GetConfig().general_.backend != "cuda") {
    std::cerr << "--device gpu needs backend = cuda in switchml.cfg" << std::endl;
    return 1;
  }

  std::cout << "Allocating and initializing data.." << std::endl;
  std::vector<int32_t> host(numel);  // float and int32 share the 4-byte storage
  uint32_t seed = f.U64("seed") ? f.U64("seed") : static_cast<uint32_t>(std::chrono::steady_clock::now().time_since_epoch().count());
  std::mt19937 rng(seed);
  // Values stay small enough that repeated in-place sums neither overflow int32 nor leave
  // the float range: |x| <= 1000 (pattern) or U(-1,1) (random).
  for (uint64_t i = 0; i < numel; i++) {
    if (is_float) {
      float v = f.Bool("random") ? std::uniform_real_distribution<float>(-1, 1)(rng)
                                 : static_cast<float>(static_cast<int>(i % 1000)) * ((i & 1) ? -1.f : 1.f);
      memcpy(&host[i], &v, 4);
    } else {
      host[i] = f.Bool("random") ? static_cast<int32_t>(rng() % 2001) - 1000
                                 : static_cast<int32_t>(i % 1000) * ((i & 1) ? -1 : 1);
    }
  }
  const std::vector<int32_t> original = host;
  void *src = host.data(), *dst = host.data();
  std::vector<int32_t> host_out;
  if (gpu) {
    cudaMalloc(&src, numel * 4);
    cudaMemcpy(src, host.data(), numel * 4, cudaMemcpyHostToDevice);
    dst = src;
    if (!inplace) cudaMalloc(&dst, numel * 4);
  } else if (!inplace) {
    host_out.resize(numel);
    dst = host_out.data();
  }
  const switchml::DataType dt = is_float ? switchml::FLOAT32 : switchml::INT32;

  auto run = [&](uint32_t jobs, bool timed, std::vector<double>& dur_ns, std::vector<double>& gbps) {
    std::vector<std::shared_ptr<switchml::Job>> pending;
    auto begin = switchml::clock::now();
    for (uint32_t i = 0; i < jobs && !g_stop; i++) {
      pending.push_back(ctx.AllReduceAsync(src, dst, numel, dt, switchml::SUM));
      if (pending.size() == sync_every || i + 1 == jobs) {
        for (auto& j : pending) j->WaitToComplete();
        auto end = switchml::clock::now();
        double ns = std::chrono::duration_cast<std::chrono::nanoseconds>(end - begin).count();
        if (timed) {
          dur_ns.push_back(ns);
          gbps.push_back(numel * 32.0 * pending.size() / ns);
          std::cout << "Job(s) #" << i + 1 - pending.size() << "-" << i << "# finished. Duration: #" << ns
                    << "# ns Goodput: #" << gbps.back() << "# Gbps." << std::endl;
          if (f.Bool("dump-stats")) {
            std::cout << ctx.GetStats().Report() << std::endl;
            ctx.GetStats().ResetStats();
          }
        }
        pending.clear();
        begin = switchml::clock::now();
      }
    }
  };
  std::vector<double> dur, gbps, unused1, unused2;
  std::cout << "Submitting " << num_warmup << " warmup jobs.." << std::endl;
  run(num_warmup, false, unused1, unused2);
  std::cout << "Warmup finished. Submitting " << num_jobs << " jobs.." << std::endl;
  run(num_jobs, true, dur, gbps);
  ctx.WaitForAllJobs();
  std::cout << "All jobs finished" << std::endl;

  int rc = 0;
  if (verify) {
    std::vector<int32_t> result(numel);
    if (gpu) cudaMemcpy(result.data(), dst, numel * 4, cudaMemcpyDeviceToHost);
    else memcpy(result.data(), dst, numel * 4);
    // In place every job multiplies by n (all workers hold the same data); out of place
    // the source never changes, so the result is always n times the input.
    double factor = inplace ? std::pow(static_cast<double>(n), num_jobs + num_warmup) : n;
    uint64_t bad = 0;
    for (uint64_t i = 0; i < numel && bad < 10; i++) {
      if (is_float) {
        float in_v, out_v;
        memcpy(&in_v, &original[i], 4);
        memcpy(&out_v, &result[i], 4);
        double want = in_v * factor;
        if (std::fabs(out_v - want) > std::fabs(want) * f.F64("err") / 100.0 + 1e-30) {
          std::cout << "data[" << i << "]: expected " << want << ", received " << out_v << std::endl;
          bad++;
        }
      } else {
        int32_t want = static_cast<int32_t>(static_cast<uint32_t>(original[i]) * static_cast<uint32_t>(std::llround(factor)));
        if (result[i] != want) {
          std::cout << "data[" << i << "]: expected " << want << ", received " << result[i] << std::endl;
          bad++;
        }
      }
    }
    std::cout << (bad ? "Failed to verify data." : "Results verified successfully.") << std::endl;
    rc = bad ? 1 : 0;
  }
  Describe("Duration", dur, "ns");
  Describe("Goodput", gbps, "Gbps");
  if (!gbps.empty()) {
    double mean_ns = std::accumulate(dur.begin(), dur.end(), 0.0) / dur.size() / sync_every;
    std::cout << "Aggregated tensor elements per second: #" << numel / (mean_ns * 1e-9) << "#" << std::endl;
  }
  ctx.Stop();
  if (gpu) {
    if (dst != src) cudaFree(dst);
    cudaFree(src);
  }
  return rc;
}
