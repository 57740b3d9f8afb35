/* Plain C interface to the library, for language bindings (Python ctypes) and for C
 * programs. Every function is thread-safe unless noted. Functions returning int return
 * 0 on success and a negative value on error (sml_last_error() has the message). */
#ifndef SWITCHML_C_H_
#define SWITCHML_C_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* data types: 0 float32, 1 int32, 2 bfloat16 (cuda backend only), 3 uint8 (summed as int32, low byte returned) */
/* job status: 0 INIT, 1 QUEUED, 2 RUNNING, 3 FINISHED, 4 FAILED */
/* context state: 0 CREATED, 1 STARTING, 2 RUNNING, 3 STOPPING, 4 STOPPED */

const char* sml_version(void);
const char* sml_last_error(void);
/* 1 if the library was compiled with -DSWITCHML_CHECKED (kernels verify their geometry). */
int sml_checked_build(void);
void sml_set_verbosity(int v);
/* per-file verbosity, "name=level,name=level" (file name without directory and extension) */
void sml_set_vmodule(const char* spec);

/* Lifecycle (switchml::Context::Start / Stop). `ini_text` is the content of a
 * switchml.cfg; NULL or "" searches the default files. apply_env != 0 lets
 * SWITCHML_RANK / SWITCHML_NUM_WORKERS / ... override the text. */
int sml_start(const char* ini_text, int apply_env);
int sml_start_file(const char* path);
int sml_stop(void);
int sml_state(void);
/* Validated configuration of the running context as INI-like text. */
int sml_config_dump(char* buf, size_t len);
/* Parse + validate without starting anything; dumps the result or returns < 0. */
int sml_config_check(const char* ini_text, char* buf, size_t len);

/* Jobs. `stream` is a cudaStream_t (NULL = default stream / host memory). Returns a
 * positive handle, or -1. Handles must be released. */
int64_t sml_allreduce_async(void* in, void* out, uint64_t numel, int dtype, void* stream);
int sml_allreduce(void* in, void* out, uint64_t numel, int dtype);
/* every worker's buffer receives the values of rank `root`; returns a job handle like
 * sml_allreduce_async (Context::BroadcastAsync) */
int64_t sml_broadcast_async(void* ptr, uint64_t numel, int dtype, int root, void* stream);
/* Wait up to timeout_ms (< 0: forever). Returns the job status. */
int sml_job_wait(int64_t job, double timeout_ms);
int sml_job_status(int64_t job);
/* Order `stream` after the job's device work without blocking the host for long. */
int sml_job_stream_wait(int64_t job, void* stream);
int sml_job_error(int64_t job, char* buf, size_t len);
void sml_job_release(int64_t job);
void sml_wait_all(void);

/* Statistics (switchml::Stats) as JSON, with backend-specific counters under "backend". */
int sml_stats_json(char* buf, size_t len);
int sml_stats_report(char* buf, size_t len);
void sml_stats_reset(void);

/* cuda backend extras */
void* sml_symm_alloc(size_t bytes);
void sml_symm_reset(void);
int sml_uses_multimem(void);
/* Bases of the symmetric heap: local, peers[0..num_workers) (room for 8), multicast. */
int sml_symm_info(void** local, void** peers, void** multicast, size_t* bytes);
int sml_device(void);
int sml_wait_probe(double budget_ms);

/* Reference arithmetic on the CPU (the oracle used by tests and --verify). */
void sml_oracle_quant_allreduce(const float* const* inputs, int num_workers, uint64_t numel,
                                uint64_t block_numel, float* out);
void sml_oracle_int_allreduce(const int32_t* const* inputs, int num_workers, uint64_t numel,
                              int32_t* out);
void sml_static_slice(uint64_t numel, int parts, int index, uint64_t* offset, uint64_t* length);

/* uint8 tensors travel as int32. widen != 0: zero-extend `numel` bytes at `in` into int32 at
 * `out`; widen == 0: keep the low byte of `numel` int32 at `in`. Device pointers of the
 * current CUDA device; the kernel is enqueued on `stream` (a cudaStream_t). */
int sml_convert_u8(int widen, const void* in, void* out, uint64_t numel, void* stream);

/* `nranks` virtual ranks on the current CUDA device in one cooperative kernel.
 * elem_type 0 f32 / 1 i32 / 2 bf16; mode 0 sum / 1 quant; algo 0 staged / 1 one-shot / 3 push;
 * exponent_lookahead: tiles by which the exponents run ahead of the data (< 0: the default). */
int sml_emu_allreduce(int nranks, void* const* in_ptrs, void* const* out_ptrs, uint64_t numel,
                      int elem_type, int mode, int algo, int block_numel, uint64_t slot_bytes,
                      int slots_per_channel, int channels, float post_scale, int repeats,
                      int exponent_lookahead);

/* Stand-alone controller / software switch (what rank 0 otherwise hosts in-process). */
void* sml_controller_start(const char* ip, int port, int udp_port);
/* the same with `pipes` data-plane threads on udp_port, udp_port + 1, ... */
void* sml_controller_start_pipes(const char* ip, int port, int udp_port, int pipes);
int sml_controller_port(void* server);
int sml_controller_udp_port(void* server);
void sml_controller_stop(void* server);
/* One CLI round trip to a controller: e.g. "SHOW statistics", "SET drop 0.01 0.01". */
int sml_controller_command(const char* ip, int port, const char* line, char* buf, size_t len);

#ifdef __cplusplus
}
#endif
#endif /* SWITCHML_C_H_ */
