// switchml_switchd: the controller and the software aggregation switch as a stand-alone
// process, for setups where no worker should host them (backend.udp.spawn_switch = false).
//
//   switchml_switchd --ip 0.0.0.0 --port 50099 --udp-port 48864 [--drop-ingress p --drop-egress p]
//                    [--log-file switchml.log] [--log-level 0..4] [--console true]
//
// With --console true the daemon also reads the console's commands from its standard input, the
// way the reference controller runs its shell in the controller process itself
// (controller/switchml.py:603-607); "exit" or end of input stops the daemon.
//
// It plays the part of the reference's controller process (controller/switchml.py:579-664:
// connect to the switch, serve the workers' session and synchronisation requests, offer a
// console) for the switch that lives in this very process. Talk to it with
// `python -m switchml_b200.utils.cli --port 50099`.
#include <signal.h>
#include <unistd.h>

#include <poll.h>

#include <atomic>
#include <cstdio>
#include <iostream>
#include <mutex>
#include <sstream>
#include <string>

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

// Console command -> request line of the control protocol ("" = not a command).
static std::string Translate(const std::string& line) {
  std::istringstream in(line);
  std::string cmd, rest;
  in >> cmd;
  std::getline(in, rest);
  static const struct { const char* name; const char* request; bool takes_args; } kTable[] = {
      {"show_ports", "SHOW ports", false},
      {"show_switch_address", "SHOW address", false},
      {"set_switch_address", "SET address", true},
      {"show_forwarding_table", "SHOW forwarding", false},
      {"show_workers", "SHOW workers", false},
      {"show_udp_workers", "SHOW workers", false},
      {"show_rdma_workers", "SHOW workers", false},
      {"show_queue_pairs_counters", "SHOW qp", false},
      {"show_bitmap", "SHOW bitmap", true},
      {"show_statistics", "SHOW statistics", false},
      {"show_slot", "SHOW slot", true},
      {"set_drop_probabilities", "SET drop", true},
      {"show_drop_probabilities", "SHOW drop", false},
      {"show_dropped_packets", "SHOW dropped", false},
      {"reset_workers", "RESET", false},
      {"ping", "PING", false},
  };
  for (const auto& e : kTable)
    if (cmd == e.name) return std::string(e.request) + (e.takes_args ? rest : "");
  return "";
}

// Serves the console on standard input until "exit", end of input or a signal.
static void Console(uint16_t port) {
  switchml::ControlClient client;
  if (!client.Connect("127.0.0.1", port, 5000)) return;
  std::cout << "(switchml) " << std::flush;
  std::string pending;
  while (g_run) {
    struct pollfd p = {0, POLLIN, 0};
    if (poll(&p, 1, 200) <= 0) continue;
    char buf[512];
    ssize_t n = read(0, buf, sizeof(buf));
    if (n <= 0) break;
    pending.append(buf, static_cast<size_t>(n));
    size_t nl;
    while ((nl = pending.find('\n')) != std::string::npos) {
      std::string line = pending.substr(0, nl);
      pending.erase(0, nl + 1);
      if (line == "exit" || line == "quit") {
        g_run = false;
        return;
      }
      if (line == "help" || line == "?") {
        std::cout << "show_ports show_switch_address set_switch_address show_forwarding_table show_workers "
                     "show_udp_workers show_rdma_workers show_queue_pairs_counters show_bitmap show_statistics "
                     "set_drop_probabilities show_drop_probabilities show_dropped_packets reset_workers ping exit\n";
      } else if (!line.empty()) {
        std::string request = Translate(line), reply;
        if (request.empty()) std::cout << "unknown command: " << line << "\n";
        else if (client.Command(request, &reply)) std::cout << reply << (reply.empty() || reply.back() == '\n' ? "" : "\n");
        else std::cout << "error\n";
      }
      std::cout << "(switchml) " << std::flush;
    }
  }
  g_run = false;
}

int main(int argc, char** argv) {
  switchml::CliFlags f;
  f.Add("ip", "0.0.0.0", "Address to listen on (TCP control and UDP data).")
      .Add("port", "50099", "TCP port of the control plane.")
      .Add("udp-port", "48864", "UDP port of the aggregation data plane (0xBEE0).")
      .Add("pipes", "4", "Data-plane threads, each with its own socket on udp-port, udp-port + 1, ... (1..8).")
      .Add("drop-ingress", "0", "Probability of dropping a packet on arrival.")
      .Add("drop-egress", "0", "Probability of dropping each result copy.")
      .Add("log-file", "switchml.log", "Also append the log to this file (empty: stderr only).")
      .Add("console", "false", "Read console commands from standard input; exit stops the daemon.")
      .Add("log-level", "1", "Verbosity 0..4.");
  if (!f.Parse(argc, argv, "SwitchML controller + software switch")) return 1;
  switchml::SetVerbosity(static_cast<int>(f.U64("log-level")));
  if (!f.Str("log-file").empty()) {
    g_log_file = fopen(f.Str("log-file").c_str(), "a");
    if (g_log_file == nullptr) std::cerr << "cannot open " << f.Str("log-file") << ", logging to stderr only\n";
    else switchml::SetLogSink(LogSink);
  }
  switchml::ControlServer server;
  if (!server.Start(f.Str("ip"), static_cast<uint16_t>(f.U64("port")), static_cast<uint16_t>(f.U64("udp-port")),
                    static_cast<int>(f.U64("pipes")))) return 1;
  server.soft_switch().SetDropProbabilities(f.F64("drop-ingress"), f.F64("drop-egress"));
  signal(SIGINT, OnSignal);
  signal(SIGTERM, OnSignal);
  std::cout << "switchml_switchd: control on " << f.Str("ip") << ":" << server.port() << ", data on UDP "
            << server.udp_port() << std::endl;
  SML_LOG(INFO) << "switchml_switchd: control on " << f.Str("ip") << ":" << server.port() << ", data on UDP "
                << server.udp_port();
  if (f.Bool("console")) Console(server.port());
  while (g_run) usleep(200 * 1000);
  std::cout << server.soft_switch().DescribeStatistics();
  server.Stop();
  SML_LOG(INFO) << "switchml_switchd stopped";
  switchml::SetLogSink(nullptr);
  if (g_log_file) fclose(g_log_file);
  return 0;
}
