// INI parser, validation and printing of the worker configuration.
// Behavioural parity with reference client_lib/src/config.cc:42-283; the parser itself
// is a small hand-written state machine keyed by "section.key".
#include "switchml/config.h"

#include <unistd.h>

#include <cmath>
#include <cstdlib>
#include <fstream>
#include <functional>
#include <sstream>
#include <vector>

#include "switchml/log.h"
#include "switchml/utils.h"

namespace switchml {

namespace {

std::string Trim(const std::string& s) {
  size_t b = s.find_first_not_of(" \t\r\n");
  if (b == std::string::npos) return "";
  size_t e = s.find_last_not_of(" \t\r\n");
  return s.substr(b, e - b + 1);
}

bool ParseBool(const std::string& v, bool* out) {
  std::string l;
  for (char c : v) l.push_back(static_cast<char>(tolower(c)));
  if (l == "true" || l == "1" || l == "yes" || l == "on") { *out = true; return true; }
  if (l == "false" || l == "0" || l == "no" || l == "off") { *out = false; return true; }
  return false;
}

template <typename T>
bool ParseUnsigned(const std::string& v, T* out) {
  if (v.empty() || v[0] == '-') return false;
  char* end = nullptr;
  unsigned long long x = strtoull(v.c_str(), &end, 0);
  if (end == v.c_str() || *end != '\0') return false;
  *out = static_cast<T>(x);
  return static_cast<unsigned long long>(*out) == x;
}

bool ParseInt(const std::string& v, int* out) {
  char* end = nullptr;
  long x = strtol(v.c_str(), &end, 0);
  if (end == v.c_str() || *end != '\0') return false;
  *out = static_cast<int>(x);
  return true;
}

bool ParseDouble(const std::string& v, double* out) {
  char* end = nullptr;
  double x = strtod(v.c_str(), &end);
  if (end == v.c_str() || *end != '\0') return false;
  *out = x;
  return true;
}

typedef std::function<bool(const std::string&)> Setter;

#define SML_OPT_UNSIGNED(field) [this](const std::string& v) { return ParseUnsigned(v, &(field)); }
#define SML_OPT_STRING(field) [this](const std::string& v) { (field) = v; return true; }
#define SML_OPT_BOOL(field) [this](const std::string& v) { return ParseBool(v, &(field)); }

}  // namespace

bool Config::LoadFromString(const std::string& text, const std::string& origin) {
  std::map<std::string, Setter> opts;
  GeneralConfig& g = general_;
  opts["general.rank"] = SML_OPT_UNSIGNED(general_.rank);
  opts["general.num_workers"] = SML_OPT_UNSIGNED(general_.num_workers);
  opts["general.num_worker_threads"] = SML_OPT_UNSIGNED(general_.num_worker_threads);
  opts["general.max_outstanding_packets"] = SML_OPT_UNSIGNED(general_.max_outstanding_packets);
  opts["general.packet_numel"] = SML_OPT_UNSIGNED(general_.packet_numel);
  opts["general.backend"] = SML_OPT_STRING(general_.backend);
  opts["general.scheduler"] = SML_OPT_STRING(general_.scheduler);
  opts["general.prepostprocessor"] = SML_OPT_STRING(general_.prepostprocessor);
  opts["general.instant_job_completion"] = SML_OPT_BOOL(general_.instant_job_completion);
  opts["general.controller_ip"] = SML_OPT_STRING(general_.controller_ip_str);
  opts["general.controller_port"] = SML_OPT_UNSIGNED(general_.controller_port);
  opts["general.timeout"] = [&g](const std::string& v) { return ParseDouble(v, &g.timeout); };
  opts["general.timeout_threshold"] = SML_OPT_UNSIGNED(general_.timeout_threshold);
  opts["general.timeout_threshold_increment"] =
      SML_OPT_UNSIGNED(general_.timeout_threshold_increment);

  opts["backend.dummy.bandwidth"] = [this](const std::string& v) {
    double d;
    if (!ParseDouble(v, &d)) return false;
    backend_.dummy.bandwidth = static_cast<float>(d);
    return true;
  };
  opts["backend.dummy.process_packets"] = SML_OPT_BOOL(backend_.dummy.process_packets);

  opts["backend.udp.switch_ip"] = SML_OPT_STRING(backend_.udp.switch_ip_str);
  opts["backend.udp.switch_port"] = SML_OPT_UNSIGNED(backend_.udp.switch_port);
  opts["backend.udp.worker_ip"] = SML_OPT_STRING(backend_.udp.worker_ip_str);
  opts["backend.udp.worker_port"] = SML_OPT_UNSIGNED(backend_.udp.worker_port);
  opts["backend.udp.spawn_switch"] = SML_OPT_BOOL(backend_.udp.spawn_switch);
  opts["backend.udp.pool_size"] = SML_OPT_UNSIGNED(backend_.udp.pool_size);
  opts["backend.udp.switch_pipes"] = SML_OPT_UNSIGNED(backend_.udp.switch_pipes);
  opts["backend.udp.cores"] = SML_OPT_STRING(backend_.udp.cores);
  opts["backend.udp.msg_numel"] = SML_OPT_UNSIGNED(backend_.udp.msg_numel);

  opts["backend.cuda.device"] = [this](const std::string& v) {
    return ParseInt(v, &backend_.cuda.device);
  };
  opts["backend.cuda.transport"] = SML_OPT_STRING(backend_.cuda.transport);
  opts["backend.cuda.mode"] = SML_OPT_STRING(backend_.cuda.mode);
  opts["backend.cuda.channels"] = SML_OPT_UNSIGNED(backend_.cuda.channels);
  opts["backend.cuda.slot_bytes"] = SML_OPT_UNSIGNED(backend_.cuda.slot_bytes);
  opts["backend.cuda.slots_per_channel"] = SML_OPT_UNSIGNED(backend_.cuda.slots_per_channel);
  opts["backend.cuda.oneshot_max_bytes"] = SML_OPT_UNSIGNED(backend_.cuda.oneshot_max_bytes);
  opts["backend.cuda.symm_heap_mb"] = SML_OPT_UNSIGNED(backend_.cuda.symm_heap_mb);
  opts["backend.cuda.average"] = SML_OPT_BOOL(backend_.cuda.average);
  opts["backend.cuda.launch"] = SML_OPT_STRING(backend_.cuda.launch);
  opts["backend.cuda.rendezvous_dir"] = SML_OPT_STRING(backend_.cuda.rendezvous_dir);
  opts["backend.cuda.p2p_algo"] = SML_OPT_STRING(backend_.cuda.p2p_algo);
  opts["backend.cuda.numa_bind"] = SML_OPT_BOOL(backend_.cuda.numa_bind);
  opts["backend.cuda.trace"] = SML_OPT_BOOL(backend_.cuda.trace);
  opts["backend.cuda.signal_fence"] = SML_OPT_STRING(backend_.cuda.signal_fence);
  opts["backend.cuda.exponent_lookahead"] = SML_OPT_UNSIGNED(backend_.cuda.exponent_lookahead);
  opts["backend.cuda.wait_timeout_ms"] = [this](const std::string& v) {
    return ParseDouble(v, &backend_.cuda.wait_timeout_ms);
  };

  std::istringstream in(text);
  std::string line, section;
  int lineno = 0;
  while (std::getline(in, line)) {
    ++lineno;
    size_t hash = line.find('#');
    if (hash != std::string::npos) line.erase(hash);
    line = Trim(line);
    if (line.empty()) continue;
    if (line.front() == '[') {
      if (line.back() != ']') {
        SML_LOG(ERROR) << origin << ":" << lineno << ": malformed section header '" << line << "'";
        return false;
      }
      section = Trim(line.substr(1, line.size() - 2));
      continue;
    }
    size_t eq = line.find('=');
    if (eq == std::string::npos) {
      SML_LOG(ERROR) << origin << ":" << lineno << ": expected 'key = value', got '" << line << "'";
      return false;
    }
    std::string key = Trim(line.substr(0, eq));
    std::string value = Trim(line.substr(eq + 1));
    std::string full = section.empty() ? key : section + "." + key;
    if (section == "backend.dpdk" || section == "backend.rdma") {
      // NIC backends of the reference have no meaning here; remember and move on.
      ignored_[full] = value;
      continue;
    }
    auto it = opts.find(full);
    if (it == opts.end()) {
      SML_LOG(ERROR) << origin << ":" << lineno << ": unrecognised option '" << full << "'";
      return false;
    }
    if (!it->second(value)) {
      SML_LOG(ERROR) << origin << ":" << lineno << ": bad value '" << value << "' for '" << full
                     << "'";
      return false;
    }
  }
  if (!ignored_.empty()) {
    SML_LOG(WARNING) << origin << ": " << ignored_.size()
                     << " option(s) of [backend.dpdk]/[backend.rdma] ignored (no NIC backends; "
                        "use backend = udp or cuda)";
  }
  loaded_from_ = origin;
  return true;
}

bool Config::LoadFromFile(std::string path) {
  std::vector<std::string> candidates;
  const char* env = getenv("SWITCHML_CONFIG");
  if (!path.empty()) {
    candidates.push_back(path);
  } else if (env && *env) {
    candidates.push_back(env);
  } else {
    char host[256] = {0};
    gethostname(host, sizeof(host) - 1);
    candidates.push_back("/etc/switchml.cfg");
    candidates.push_back("./switchml.cfg");
    candidates.push_back(std::string("./switchml-") + host + ".cfg");
  }
  for (const std::string& c : candidates) {
    std::ifstream f(c);
    if (!f.good()) continue;
    std::stringstream buf;
    buf << f.rdbuf();
    SML_VLOG(1) << "Loading configuration from '" << c << "'";
    return LoadFromString(buf.str(), c);
  }
  std::string tried;
  for (const std::string& c : candidates) tried += " " + c;
  SML_LOG(ERROR) << "No configuration file found; tried:" << tried;
  return false;
}

void Config::ApplyEnvOverrides() {
  const char* e;
  if ((e = getenv("SWITCHML_RANK")) && *e) ParseUnsigned(std::string(e), &general_.rank);
  if ((e = getenv("SWITCHML_NUM_WORKERS")) && *e)
    ParseUnsigned(std::string(e), &general_.num_workers);
  if ((e = getenv("SWITCHML_BACKEND")) && *e) general_.backend = e;
  if ((e = getenv("SWITCHML_CONTROLLER_PORT")) && *e)
    ParseUnsigned(std::string(e), &general_.controller_port);
}

static bool IsPow2(uint64_t x) { return x && !(x & (x - 1)); }

void Config::Validate() {
  GeneralConfig& g = general_;
  SML_CHECK(g.num_workers >= 1 && g.num_workers <= 32)
      << "num_workers must be in [1,32], got " << g.num_workers;
  SML_CHECK(g.rank < g.num_workers) << "rank " << g.rank << " is not below num_workers "
                                    << g.num_workers;
  SML_CHECK(g.num_worker_threads >= 1) << "num_worker_threads must be at least 1";
  SML_CHECK(g.packet_numel >= 1) << "packet_numel must be at least 1";
  SML_CHECK(g.scheduler == "fifo") << "'" << g.scheduler << "' is not a valid scheduler";
  SML_CHECK(g.prepostprocessor == "cpu_exponent_quantizer" || g.prepostprocessor == "bypass")
      << "'" << g.prepostprocessor << "' is not a valid prepostprocessor";
  SML_CHECK(g.backend == "dummy" || g.backend == "udp" || g.backend == "cuda")
      << "'" << g.backend << "' is not a valid backend (dummy | udp | cuda)";

  // Every worker thread needs at least one slot, and the window divides evenly.
  SML_CHECK(g.max_outstanding_packets >= g.num_worker_threads)
      << "max_outstanding_packets (" << g.max_outstanding_packets
      << ") must be at least num_worker_threads (" << g.num_worker_threads << ")";
  if (g.max_outstanding_packets % g.num_worker_threads != 0) {
    uint32_t t = g.num_worker_threads;
    uint32_t rounded = static_cast<uint32_t>(
        std::lround(static_cast<double>(g.max_outstanding_packets) / t)) * t;
    if (rounded < t) rounded = t;
    SML_LOG(WARNING) << "max_outstanding_packets " << g.max_outstanding_packets
                     << " is not a multiple of num_worker_threads " << t << "; using " << rounded;
    g.max_outstanding_packets = rounded;
  }
  SML_CHECK(g.timeout > 0) << "timeout must be positive";

  if (g.backend == "udp") {
    SML_CHECK(g.packet_numel == 64 || g.packet_numel == 256)
        << "the udp backend supports packet_numel 64 or 256, got " << g.packet_numel;
    SML_CHECK(g.max_outstanding_packets / g.num_worker_threads <= backend_.udp.pool_size)
        << "window per worker thread exceeds backend.udp.pool_size";
    SML_CHECK(g.max_outstanding_packets <= 16384) << "the software switch has 16384 slots";
    // Messages of several packets (the reference's backend.rdma.msg_numel, config.cc:185-211):
    // a whole number of packets per message, a whole number of messages per worker thread.
    UdpBackendConfig& u = backend_.udp;
    if (u.msg_numel == 0) u.msg_numel = g.packet_numel;
    SML_CHECK(u.msg_numel >= g.packet_numel) << "backend.udp.msg_numel cannot be less than general.packet_numel";
    if (u.msg_numel % g.packet_numel != 0) {
      uint32_t rounded = u.msg_numel / g.packet_numel * g.packet_numel;
      SML_LOG(WARNING) << "backend.udp.msg_numel " << u.msg_numel << " is not divisible by general.packet_numel "
                       << g.packet_numel << "; using " << rounded;
      u.msg_numel = rounded;
    }
    const uint32_t pkts_per_msg = u.msg_numel / g.packet_numel;
    SML_CHECK(pkts_per_msg <= 64) << "backend.udp.msg_numel: at most 64 packets per message";
    const uint32_t per_round = g.num_worker_threads * pkts_per_msg;
    if (g.max_outstanding_packets % per_round != 0) {
      // the nearer of the two neighbouring multiples, never less than one message per thread
      uint32_t lower = g.max_outstanding_packets / per_round * per_round, upper = lower + per_round;
      uint32_t chosen = (lower >= per_round && g.max_outstanding_packets - lower <= upper - g.max_outstanding_packets) ? lower : upper;
      SML_LOG(WARNING) << "max_outstanding_packets " << g.max_outstanding_packets << " is not divisible by " << per_round
                       << " (packets per message x worker threads); using " << chosen << " to have exactly "
                       << chosen / per_round << " outstanding messages per worker thread";
      g.max_outstanding_packets = chosen;
      SML_CHECK(g.max_outstanding_packets <= 16384 && g.max_outstanding_packets / g.num_worker_threads <= u.pool_size)
          << "max_outstanding_packets after rounding to whole messages exceeds the switch pool";
    }
    SML_CHECK(backend_.udp.switch_pipes <= 8) << "backend.udp.switch_pipes must be between 0 (automatic) and 8";
    if (!backend_.udp.cores.empty()) {
      int ids[256], count = 0;
      std::string err;
      SML_CHECK(ParseCoreList(backend_.udp.cores, &err, ids, 256, &count))
          << "backend.udp.cores: " << err;
      SML_CHECK(count >= g.num_worker_threads)
          << "backend.udp.cores names " << count << " core(s) for " << g.num_worker_threads
          << " worker threads";
    }
  }
  if (g.backend == "cuda") {
    CudaBackendConfig& c = backend_.cuda;
    SML_CHECK(IsPow2(g.packet_numel) && g.packet_numel >= 32 && g.packet_numel <= 1024)
        << "the cuda backend needs packet_numel to be a power of two in [32,1024], got "
        << g.packet_numel;
    SML_CHECK(c.transport == "auto" || c.transport == "nvls" || c.transport == "p2p")
        << "backend.cuda.transport must be auto | nvls | p2p";
    SML_CHECK(c.mode == "int32_quant" || c.mode == "float_sum")
        << "backend.cuda.mode must be int32_quant | float_sum";
    SML_CHECK(c.p2p_algo == "push" || c.p2p_algo == "staged")
        << "backend.cuda.p2p_algo must be push | staged";
    SML_CHECK(c.launch == "worker" || c.launch == "inline")
        << "backend.cuda.launch must be worker | inline";
    SML_CHECK(c.slots_per_channel >= 1 && c.slots_per_channel <= 8)
        << "backend.cuda.slots_per_channel must be in [1,8]";
    SML_CHECK(c.channels <= 512) << "backend.cuda.channels must be at most 512";
    SML_CHECK(c.signal_fence == "sc" || c.signal_fence == "release")
        << "backend.cuda.signal_fence must be sc | release";
    SML_CHECK(c.exponent_lookahead <= 4) << "backend.cuda.exponent_lookahead must be in [0,4]";
    // A slot is cut into num_workers shards of whole quantisation blocks, so its length
    // must be a multiple of num_workers * packet_numel elements (4 bytes each); keep the
    // shards 16-byte vectorisable as well.
    uint64_t quantum = static_cast<uint64_t>(g.num_workers) * (g.packet_numel > 128 ? g.packet_numel : 128) * 4;
    if (c.slot_bytes < quantum) c.slot_bytes = quantum;
    if (c.slot_bytes % quantum != 0) {
      uint64_t rounded = (c.slot_bytes / quantum) * quantum;
      SML_LOG(WARNING) << "backend.cuda.slot_bytes " << c.slot_bytes << " rounded down to "
                       << rounded << " (multiple of num_workers*max(packet_numel,128)*4)";
      c.slot_bytes = rounded;
    }
    // The scale factors of all slots of a channel live in shared memory (8192 floats).
    uint64_t max_slot = 8192ull / c.slots_per_channel * g.packet_numel * 4 / quantum * quantum;
    SML_CHECK(max_slot >= quantum) << "backend.cuda: packet_numel too small for " << c.slots_per_channel
                                   << " slots per channel";
    if (c.slot_bytes > max_slot) {
      SML_VLOG(1) << "backend.cuda.slot_bytes lowered from " << c.slot_bytes << " to " << max_slot
                  << " (at most 8192 quantisation blocks over a channel's slots)";
      c.slot_bytes = max_slot;
    }
    SML_CHECK(c.wait_timeout_ms > 0) << "backend.cuda.wait_timeout_ms must be positive";
    SML_CHECK(g.num_workers <= 8) << "the cuda backend serves at most 8 GPUs (one NVSwitch domain)";
  }
}

std::string Config::ToString() const {
  const GeneralConfig& g = general_;
  std::ostringstream o;
  o << "[general]\n"
    << "    rank = " << g.rank << "\n"
    << "    num_workers = " << g.num_workers << "\n"
    << "    num_worker_threads = " << g.num_worker_threads << "\n"
    << "    max_outstanding_packets = " << g.max_outstanding_packets << "\n"
    << "    packet_numel = " << g.packet_numel << "\n"
    << "    backend = " << g.backend << "\n"
    << "    scheduler = " << g.scheduler << "\n"
    << "    prepostprocessor = " << g.prepostprocessor << "\n"
    << "    instant_job_completion = " << (g.instant_job_completion ? "true" : "false") << "\n"
    << "    controller_ip = " << g.controller_ip_str << "\n"
    << "    controller_port = " << g.controller_port << "\n"
    << "    timeout = " << g.timeout << "\n"
    << "    timeout_threshold = " << g.timeout_threshold << "\n"
    << "    timeout_threshold_increment = " << g.timeout_threshold_increment << "\n"
    << "  (derived)\n"
    << "    outstanding packets per worker thread = "
    << g.max_outstanding_packets / (g.num_worker_threads ? g.num_worker_threads : 1) << "\n"
    << "    packet payload bytes = " << g.packet_numel * 4 << "\n"
    << "    bytes in flight per worker = " << g.packet_numel * 4 * g.max_outstanding_packets
    << "\n";
  if (g.backend == "dummy") {
    o << "[backend.dummy]\n"
      << "    bandwidth = " << backend_.dummy.bandwidth << "\n"
      << "    process_packets = " << (backend_.dummy.process_packets ? "true" : "false") << "\n";
  } else if (g.backend == "udp") {
    const UdpBackendConfig& u = backend_.udp;
    o << "[backend.udp]\n"
      << "    switch_ip = " << u.switch_ip_str << "\n"
      << "    switch_port = " << u.switch_port << "\n"
      << "    worker_ip = " << u.worker_ip_str << "\n"
      << "    worker_port = " << u.worker_port << "\n"
      << "    spawn_switch = " << (u.spawn_switch ? "true" : "false") << "\n"
      << "    pool_size = " << u.pool_size << "\n"
      << "    switch_pipes = " << u.switch_pipes << "\n"
      << "    cores = " << u.cores << "\n"
      << "    msg_numel = " << u.msg_numel << "\n";
  } else if (g.backend == "cuda") {
    const CudaBackendConfig& c = backend_.cuda;
    o << "[backend.cuda]\n"
      << "    device = " << c.device << "\n"
      << "    transport = " << c.transport << "\n"
      << "    mode = " << c.mode << "\n"
      << "    channels = " << c.channels << "\n"
      << "    slot_bytes = " << c.slot_bytes << "\n"
      << "    slots_per_channel = " << c.slots_per_channel << "\n"
      << "    oneshot_max_bytes = " << c.oneshot_max_bytes << "\n"
      << "    symm_heap_mb = " << c.symm_heap_mb << "\n"
      << "    average = " << (c.average ? "true" : "false") << "\n"
      << "    launch = " << c.launch << "\n"
      << "    rendezvous_dir = " << c.rendezvous_dir << "\n"
      << "    wait_timeout_ms = " << c.wait_timeout_ms << "\n"
      << "    numa_bind = " << (c.numa_bind ? "true" : "false") << "\n"
      << "    p2p_algo = " << c.p2p_algo << "\n"
      << "    exponent_lookahead = " << c.exponent_lookahead << "\n"
      << "    signal_fence = " << c.signal_fence << "\n"
      << "    trace = " << (c.trace ? "true" : "false") << "\n";
  }
  for (const auto& kv : ignored_) o << "  (ignored) " << kv.first << " = " << kv.second << "\n";
  return o.str();
}

void Config::PrintConfig() const {
  SML_VLOG(1) << "Printing configuration"
              << (loaded_from_.empty() ? std::string() : " (" + loaded_from_ + ")") << "\n"
              << ToString();
}

}  // namespace switchml
