// switchml_switchd: the controller and the software aggregation switch as a stand-alone
// process, for setups where no worker should host them (backend.udp.spawn_switch = false).
//
//   switchml_switchd --ip 0.0.0.0 --port 50099 --udp-port 48864 [--drop-ingress p --drop-egress p]
//                    [--log-file switchml.log] [--log-level 0..4]
//
// It plays the part of the reference's controller process (controller/switchml.py:579-664:
// connect to the switch, serve the workers' session and synchronisation requests, offer a
// console) for the switch that lives in this very process. Talk to it with
// `python -m switchml_b200.utils.cli --port 50099`.
#include <signal.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <iostream>
#include <mutex>

#include "rendezvous/control.h"
#include "switchml/cli_flags.h"
#include "switchml/log.h"

static std::atomic<bool> g_run{true};
static void OnSignal(int) { g_run = false; }

// Log lines go to stderr and, like the reference controller's switchml.log
// (controller/switchml.py:659-664), to a file.
static FILE* g_log_file = nullptr;
static std::mutex g_log_mu;
static void LogSink(int severity, const char* line) {
  std::lock_guard<std::mutex> lk(g_log_mu);
  fprintf(stderr, "%s\n", line);
  if (g_log_file) {
    fprintf(g_log_file, "%s\n", line);
    fflush(g_log_file);
  }
}

int main(int argc, char** argv) {
  switchml::CliFlags f;
  f.Add("ip", "0.0.0.0", "Address to listen on (TCP control and UDP data).")
      .Add("port", "50099", "TCP port of the control plane.")
      .Add("udp-port", "48864", "UDP port of the aggregation data plane (0xBEE0).")
      .Add("drop-ingress", "0", "Probability of dropping a packet on arrival.")
      .Add("drop-egress", "0", "Probability of dropping each result copy.")
      .Add("log-file", "switchml.log", "Also append the log to this file (empty: stderr only).")
      .Add("log-level", "1", "Verbosity 0..4.");
  if (!f.Parse(argc, argv, "SwitchML controller + software switch")) return 1;
  switchml::SetVerbosity(static_cast<int>(f.U64("log-level")));
  if (!f.Str("log-file").empty()) {
    g_log_file = fopen(f.Str("log-file").c_str(), "a");
    if (g_log_file == nullptr) std::cerr << "cannot open " << f.Str("log-file") << ", logging to stderr only\n";
    else switchml::SetLogSink(LogSink);
  }
  switchml::ControlServer server;
  if (!server.Start(f.Str("ip"), static_cast<uint16_t>(f.U64("port")), static_cast<uint16_t>(f.U64("udp-port")))) return 1;
  server.soft_switch().SetDropProbabilities(f.F64("drop-ingress"), f.F64("drop-egress"));
  signal(SIGINT, OnSignal);
  signal(SIGTERM, OnSignal);
  std::cout << "switchml_switchd: control on " << f.Str("ip") << ":" << server.port() << ", data on UDP "
            << server.udp_port() << std::endl;
  SML_LOG(INFO) << "switchml_switchd: control on " << f.Str("ip") << ":" << server.port() << ", data on UDP "
                << server.udp_port();
  while (g_run) usleep(200 * 1000);
  std::cout << server.soft_switch().DescribeStatistics();
  server.Stop();
  SML_LOG(INFO) << "switchml_switchd stopped";
  switchml::SetLogSink(nullptr);
  if (g_log_file) fclose(g_log_file);
  return 0;
}
