// Shared host-side plumbing of the library: context, thread-local error state,
// host<->device staging for the reference's host-pointer calling convention.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/exo_b200.h"

namespace exob200 {

constexpr uint32_t kContextMagic = 0x45584F42u;  // "EXOB"

// Device-side status word written by kernels whose bounded waits ran out.
struct DeviceStatus {
  int code;      // 0 = ok, otherwise EXO_B200_ERR_*
  int where;     // kernel-specific location id
  int block;     // blockIdx.x that gave up first
  int detail;
};

}  // namespace exob200

struct exo_b200_Context {
  uint32_t magic;
  int device;
  cudaStream_t stream;
  int sgemm_path;
  int sm_count;
  // grow-only device staging area for host-pointer calls
  void* stage[4];
  size_t stage_bytes[4];
  // device scratch for kernels that need it (repacked operands)
  void* scratch[2];
  size_t scratch_bytes[2];
  exob200::DeviceStatus* status_dev;   // device word
  exob200::DeviceStatus* status_host;  // pinned mirror
};

namespace exob200 {

void set_error(int code, const std::string& msg);
void clear_error();
int last_error_code();
const char* last_error_msg();
bool check_cuda(cudaError_t e, const char* what);

// Resolves ctxt (NULL or a pointer made by exo_b200_context_create) to a
// usable context on an sm_100 device, or returns nullptr with the error set.
exo_b200_Context* resolve_context(void* ctxt);
exo_b200_Context* default_context();

// true if p is device-accessible memory (device or managed allocation)
bool is_device_pointer(const void* p);

// One operand of a call.  For host memory, `dev` points into the context's
// staging area; inputs are copied in before the launch, outputs copied back
// after it.
struct Operand {
  const void* user;
  void* dev;
  size_t bytes;
  bool staged;
};

// Prepares operand `slot` (0..3).  copy_in: contents are needed on the device.
bool stage_in(exo_b200_Context* c, int slot, const void* user, size_t bytes, bool copy_in, Operand* op);
// Copies a staged output back and synchronises; no-op for device pointers.
bool stage_out(exo_b200_Context* c, const Operand& op);
// If any operand was staged the call is synchronous: wait and read the status.
bool finish(exo_b200_Context* c, bool any_staged);

bool ensure_scratch(exo_b200_Context* c, int slot, size_t bytes);

}  // namespace exob200
