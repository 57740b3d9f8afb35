// Passing file descriptors between the worker processes of one machine.
//
// Memory handles exported by the CUDA driver are POSIX file descriptors; a descriptor
// only has meaning inside its process, so it travels as SCM_RIGHTS ancillary data over a
// unix-domain socket. Each rank listens on a socket named after the session and its rank
// (Linux abstract namespace by default, or a path under `dir`).
#ifndef SWITCHML_CUDA_FD_CHANNEL_H_
#define SWITCHML_CUDA_FD_CHANNEL_H_

#include <cstdint>
#include <string>

namespace switchml {

class FdChannel {
 public:
  FdChannel();
  ~FdChannel();
  // Start listening as `rank` of session `session_id`.
  bool Listen(uint64_t session_id, int rank, const std::string& dir);
  // Send `fd` to `peer`, labelled with (`from_rank`, `tag`).
  bool SendTo(int peer, int from_rank, int tag, int fd);
  // Receive one descriptor; fills who sent it and its tag. Waits up to `timeout_ms`.
  bool Recv(int* from_rank, int* tag, int* fd, int timeout_ms = 30000);
  void Close();

 private:
  std::string Name(int rank) const;
  int listen_fd_ = -1;
  uint64_t session_id_ = 0;
  std::string dir_;
  std::string bound_path_;
};

}  // namespace switchml
#endif  // SWITCHML_CUDA_FD_CHANNEL_H_
