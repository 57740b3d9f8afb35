// See fd_channel.h.
#include "backends/cuda/fd_channel.h"

#include <errno.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cstring>

#include "switchml/log.h"

namespace switchml {

FdChannel::FdChannel() {}
FdChannel::~FdChannel() { Close(); }

std::string FdChannel::Name(int rank) const {
  std::string base = "switchml-" + std::to_string(session_id_) + "-" + std::to_string(rank);
  return dir_.empty() ? base : dir_ + "/" + base + ".sock";
}

static socklen_t FillAddr(const std::string& name, bool abstract_ns, sockaddr_un* a) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  if (abstract_ns) {
    // Abstract namespace: leading NUL, no file system entry, vanishes with the process.
    size_t n = name.size() < sizeof(a->sun_path) - 2 ? name.size() : sizeof(a->sun_path) - 2;
    memcpy(a->sun_path + 1, name.data(), n);
    return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
  }
  strncpy(a->sun_path, name.c_str(), sizeof(a->sun_path) - 1);
  return sizeof(*a);
}

bool FdChannel::Listen(uint64_t session_id, int rank, const std::string& dir) {
  session_id_ = session_id;
  dir_ = dir;
  listen_fd_ = socket(AF_UNIX, SOCK_STREAM, 0);
  if (listen_fd_ < 0) return false;
  sockaddr_un a;
  std::string name = Name(rank);
  socklen_t len = FillAddr(name, dir_.empty(), &a);
  if (!dir_.empty()) {
    unlink(name.c_str());
    bound_path_ = name;
  }
  if (bind(listen_fd_, reinterpret_cast<sockaddr*>(&a), len) != 0 || listen(listen_fd_, 64) != 0) {
    SML_LOG(ERROR) << "fd channel: cannot listen on '" << name << "': " << strerror(errno);
    close(listen_fd_);
    listen_fd_ = -1;
    return false;
  }
  return true;
}

bool FdChannel::SendTo(int peer, int from_rank, int tag, int fd) {
  int s = socket(AF_UNIX, SOCK_STREAM, 0);
  if (s < 0) return false;
  sockaddr_un a;
  socklen_t len = FillAddr(Name(peer), dir_.empty(), &a);
  bool ok = false;
  for (int attempt = 0; attempt < 200; attempt++) {
    if (connect(s, reinterpret_cast<sockaddr*>(&a), len) == 0) { ok = true; break; }
    usleep(10 * 1000);
  }
  if (!ok) {
    SML_LOG(ERROR) << "fd channel: cannot connect to rank " << peer << ": " << strerror(errno);
    close(s);
    return false;
  }
  int32_t meta[2] = {from_rank, tag};
  struct iovec iov = {meta, sizeof(meta)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  ok = sendmsg(s, &msg, 0) == static_cast<ssize_t>(sizeof(meta));
  // The kernel holds its own reference to the descriptor while the message is queued,
  // so closing right away is safe and nobody has to be receiving yet.
  close(s);
  return ok;
}

bool FdChannel::Recv(int* from_rank, int* tag, int* fd, int timeout_ms) {
  struct pollfd p = {listen_fd_, POLLIN, 0};
  if (poll(&p, 1, timeout_ms) <= 0) return false;
  int s = accept(listen_fd_, nullptr, nullptr);
  if (s < 0) return false;
  int32_t meta[2] = {0, 0};
  struct iovec iov = {meta, sizeof(meta)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  bool ok = recvmsg(s, &msg, 0) == static_cast<ssize_t>(sizeof(meta));
  struct cmsghdr* c = ok ? CMSG_FIRSTHDR(&msg) : nullptr;
  if (c && c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
    memcpy(fd, CMSG_DATA(c), sizeof(int));
    *from_rank = meta[0];
    *tag = meta[1];
  } else {
    ok = false;
  }
  close(s);
  return ok;
}

void FdChannel::Close() {
  if (listen_fd_ >= 0) close(listen_fd_);
  listen_fd_ = -1;
  if (!bound_path_.empty()) unlink(bound_path_.c_str());
  bound_path_.clear();
}

}  // namespace switchml
