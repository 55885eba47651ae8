// Shared host-side plumbing of the library: context, thread-local error state,
// host<->device staging for the reference's host-pointer calling convention.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <vector>

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

namespace exob200 {
// identity of a weight tensor whose TF32 split is held in the context (tensor-core convolution)
struct WeightKey {
  const void* ptr;
  int in_c, out_c, kdim;
  int64_t stride_ky, stride_kx, stride_ci;
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
  void* scratch[3];  // 0, 1: per-call operand copies; 2: the split weights of the tensor-core convolution
  size_t scratch_bytes[3];
  // Each scratch slot remembers the stream of its last user and an event recorded after the
  // last kernel that reads it, so that a call on ANOTHER stream waits for that reader before
  // its pre-pass overwrites the slot (calls on one stream are ordered anyway).
  cudaEvent_t scratch_ev[3];
  cudaStream_t scratch_stream[3];
  bool scratch_busy[3];
  // weight cache (off unless exo_b200_context_cache_weights switched it on)
  bool cache_weights, wkey_valid;
  exob200::WeightKey wkey;
  // resident CTA pairs of the two cluster kernels on this context's device (0 = not asked yet)
  int max_pairs[4];
  exob200::DeviceStatus* status_dev;   // device word
  exob200::DeviceStatus* status_host;  // pinned mirror
  // host-pointer row pipeline: copy-in / copy-out streams, two chunk buffers each way
  cudaStream_t pipe_in, pipe_out;
  cudaEvent_t ev_in[2], ev_kernel[2], ev_out[2], ev_ready;
  void* pipe_a[2];
  void* pipe_c[2];
  size_t pipe_a_bytes, pipe_c_bytes;
  bool pipe_ready;
  // host-pointer block pipeline: ring of dense C blocks and the events that guard them
  void* blk_c[4];
  size_t blk_c_bytes;
  cudaEvent_t ev_blk_kernel[4], ev_blk_out[4], ev_upload;
  bool blk_ready;
  bool is_default;              // the per-device context that ctxt == NULL resolves to
  std::recursive_mutex* mutex;  // held by an entry point for the whole call (staging and scratch are shared)
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

// Holds the context's mutex for the scope of one entry-point call, so that host threads
// calling into one context (in particular the shared default context, as OpenMP callers of
// the generated C would) take turns with its staging buffers, scratch and pipeline.  For the
// default context it also installs the calling thread's default stream.
class ContextUse {
 public:
  explicit ContextUse(exo_b200_Context* c);
  ~ContextUse();
  ContextUse(const ContextUse&) = delete;
  ContextUse& operator=(const ContextUse&) = delete;
  exo_b200_Context* get() const { return c_; }

 private:
  exo_b200_Context* c_;
  int restore_device_;  // >= 0: the device that was current before this call
};

// true if p is device-accessible memory (device or managed allocation)
bool is_device_pointer(const void* p);
// Device ordinal that owns p if p is a plain device allocation, -1 otherwise (host, managed, unknown).
int owning_device(const void* p);

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
// Scratch slot `slot`, at least `bytes` large, safe to overwrite from c->stream: if the slot's
// last reader ran on a different stream, c->stream is made to wait for it first.
bool acquire_scratch(exo_b200_Context* c, int slot, size_t bytes);
// To be called after the last kernel that reads the slot has been enqueued on c->stream.
void release_scratch(exo_b200_Context* c, int slot);

// Host-pointer calls whose output rows depend only on the matching rows of one
// input (GEMM: C rows <- A rows) are run as a pipeline over row chunks: while
// chunk i is multiplied, chunk i+1 is copied in and chunk i-1 is copied out on
// two side streams, so the PCIe copies in both directions overlap each other and
// the kernels instead of adding up.  `launch(rows, dA, dC)` enqueues the kernel
// for one chunk on c->stream.  Returns false with the error set on failure; on
// return all copies have completed.
struct RowPipeline {
  int64_t rows;            // total rows
  int64_t chunk_rows;      // rows per chunk
  const void* host_a;      // row-major, a_row_bytes per row
  size_t a_row_bytes;
  void* host_c;
  size_t c_row_bytes;
  bool c_is_input;         // C is read by the kernel (C += ...): copy it in too
};
bool pipeline_prepare(exo_b200_Context* c, size_t a_chunk_bytes, size_t c_chunk_bytes);

// The same idea in two dimensions, for products whose second operand is also on the
// host and large: C[i-th row chunk, j-th column block] needs only row chunk i of the
// first operand and column block j of the second, so waiting for all of the second
// operand before the first output can leave (as the row pipeline does) is not
// necessary.  Both operands are uploaded piecewise in the order that enables the most
// output bytes per uploaded byte; every block that becomes computable is multiplied
// into a dense block buffer and copied out as a strided 2-D copy.  `launch(rows, cols,
// dA, dB, dC)` enqueues the kernel for one block (dC dense, pitch = cols) on c->stream.
struct BlockPipeline {
  int64_t rows, cols;              // C is rows x cols, row-major
  int64_t chunk_rows, chunk_cols;  // block size
  const void* host_a;              // rows x a_row_bytes
  size_t a_row_bytes;
  const void* host_b;              // cols x b_col_bytes: column j of the product's second operand is contiguous
  size_t b_col_bytes;
  void* host_c;
  size_t c_elem_bytes;
};
bool block_pipeline_prepare(exo_b200_Context* c, size_t a_bytes, size_t b_bytes, size_t c_block_bytes);
// The upload order: 'A' / 'B' per step, chosen greedily by output bytes enabled per byte uploaded.
std::vector<char> block_upload_order(const BlockPipeline& p);

template <class Launch>
bool run_block_pipeline_impl(exo_b200_Context* c, const BlockPipeline& p, Launch launch);
template <class Launch>
bool run_block_pipeline(exo_b200_Context* c, const BlockPipeline& p, Launch launch) {
  if (run_block_pipeline_impl(c, p, launch)) return true;
  const int code = last_error_code();
  const std::string msg = last_error_msg();
  cudaStreamSynchronize(c->stream);
  if (c->pipe_ready) {
    cudaStreamSynchronize(c->pipe_in);
    cudaStreamSynchronize(c->pipe_out);
  }
  cudaGetLastError();
  set_error(code, msg);
  return false;
}

template <class Launch>
bool run_block_pipeline_impl(exo_b200_Context* c, const BlockPipeline& p, Launch launch) {
  const int64_t na = (p.rows + p.chunk_rows - 1) / p.chunk_rows, nb = (p.cols + p.chunk_cols - 1) / p.chunk_cols;
  const size_t blk_bytes = (size_t)p.chunk_rows * p.chunk_cols * p.c_elem_bytes;
  if (!block_pipeline_prepare(c, (size_t)p.rows * p.a_row_bytes, (size_t)p.cols * p.b_col_bytes, blk_bytes))
    return false;
  char* dA = static_cast<char*>(c->stage[0]);
  char* dB = static_cast<char*>(c->stage[1]);
  // work enqueued earlier on c->stream may still read the staging buffers
  if (!check_cuda(cudaEventRecord(c->ev_ready, c->stream), "cudaEventRecord")) return false;
  cudaStreamWaitEvent(c->pipe_in, c->ev_ready, 0);
  cudaStreamWaitEvent(c->pipe_out, c->ev_ready, 0);
  auto rows_of = [&](int64_t i) { return std::min(p.chunk_rows, p.rows - i * p.chunk_rows); };
  auto cols_of = [&](int64_t j) { return std::min(p.chunk_cols, p.cols - j * p.chunk_cols); };
  int64_t a_done = 0, b_done = 0, nblk = 0;
  auto run_block = [&](int64_t i, int64_t j) -> bool {
    const int buf = (int)(nblk & 3);
    if (nblk >= 4) cudaStreamWaitEvent(c->stream, c->ev_blk_out[buf], 0);  // its last copy-out has drained
    const int64_t r = rows_of(i), w = cols_of(j);
    if (!check_cuda(launch(r, w, dA + (size_t)i * p.chunk_rows * p.a_row_bytes,
                           dB + (size_t)j * p.chunk_cols * p.b_col_bytes, c->blk_c[buf]),
                    "block kernel"))
      return false;
    cudaEventRecord(c->ev_blk_kernel[buf], c->stream);
    cudaStreamWaitEvent(c->pipe_out, c->ev_blk_kernel[buf], 0);
    char* hc = static_cast<char*>(p.host_c) +
               ((size_t)i * p.chunk_rows * p.cols + (size_t)j * p.chunk_cols) * p.c_elem_bytes;
    if (!check_cuda(cudaMemcpy2DAsync(hc, (size_t)p.cols * p.c_elem_bytes, c->blk_c[buf], (size_t)w * p.c_elem_bytes,
                                      (size_t)w * p.c_elem_bytes, (size_t)r, cudaMemcpyDeviceToHost, c->pipe_out),
                    "D2H block"))
      return false;
    cudaEventRecord(c->ev_blk_out[buf], c->pipe_out);
    nblk++;
    return true;
  };
  for (char step : block_upload_order(p)) {
    if (step == 'A') {
      const size_t off = (size_t)a_done * p.chunk_rows * p.a_row_bytes;
      if (!check_cuda(cudaMemcpyAsync(dA + off, static_cast<const char*>(p.host_a) + off,
                                      (size_t)rows_of(a_done) * p.a_row_bytes, cudaMemcpyHostToDevice, c->pipe_in),
                      "H2D chunk"))
        return false;
    } else {
      const size_t off = (size_t)b_done * p.chunk_cols * p.b_col_bytes;
      if (!check_cuda(cudaMemcpyAsync(dB + off, static_cast<const char*>(p.host_b) + off,
                                      (size_t)cols_of(b_done) * p.b_col_bytes, cudaMemcpyHostToDevice, c->pipe_in),
                      "H2D chunk"))
        return false;
    }
    // the copy stream is in order: this event also covers every earlier piece.  It is
    // re-recorded per step, which is safe because the wait below is enqueued first.
    cudaEventRecord(c->ev_upload, c->pipe_in);
    cudaStreamWaitEvent(c->stream, c->ev_upload, 0);
    if (step == 'A') {
      for (int64_t j = 0; j < b_done; j++)
        if (!run_block(a_done, j)) return false;
      a_done++;
    } else {
      for (int64_t i = 0; i < a_done; i++)
        if (!run_block(i, b_done)) return false;
      b_done++;
    }
  }
  if (!check_cuda(cudaStreamSynchronize(c->pipe_out), "cudaStreamSynchronize")) return false;
  if (!check_cuda(cudaStreamSynchronize(c->pipe_in), "cudaStreamSynchronize")) return false;
  if (nblk != na * nb) {
    set_error(EXO_B200_ERR_CUDA, "block pipeline: not every output block was scheduled");
    return false;
  }
  return true;
}


// On any failure the copies already enqueued may still be writing the caller's buffers:
// drain the three streams before reporting it.
inline void pipeline_drain(exo_b200_Context* c) {
  if (c->pipe_ready) {
    cudaStreamSynchronize(c->pipe_in);
    cudaStreamSynchronize(c->pipe_out);
  }
  cudaStreamSynchronize(c->stream);
}

template <class Launch>
bool run_row_pipeline_impl(exo_b200_Context* c, const RowPipeline& p, Launch launch);
template <class Launch>
bool run_row_pipeline(exo_b200_Context* c, const RowPipeline& p, Launch launch) {
  if (run_row_pipeline_impl(c, p, launch)) return true;
  const int code = last_error_code();
  const std::string msg = last_error_msg();
  pipeline_drain(c);
  cudaGetLastError();
  set_error(code, msg);
  return false;
}

template <class Launch>
bool run_row_pipeline_impl(exo_b200_Context* c, const RowPipeline& p, Launch launch) {
  const size_t a_chunk = (size_t)p.chunk_rows * p.a_row_bytes, c_chunk = (size_t)p.chunk_rows * p.c_row_bytes;
  if (!pipeline_prepare(c, a_chunk, c_chunk)) return false;
  // everything enqueued on c->stream so far (the staged B operand) must be in place first
  if (!check_cuda(cudaEventRecord(c->ev_ready, c->stream), "cudaEventRecord")) return false;
  const int64_t nchunks = (p.rows + p.chunk_rows - 1) / p.chunk_rows;
  for (int64_t i = 0; i < nchunks; i++) {
    const int b = (int)(i & 1);
    const int64_t r0 = i * p.chunk_rows;
    const int64_t rows = p.rows - r0 < p.chunk_rows ? p.rows - r0 : p.chunk_rows;
    const char* ha = static_cast<const char*>(p.host_a) + (size_t)r0 * p.a_row_bytes;
    char* hc = static_cast<char*>(p.host_c) + (size_t)r0 * p.c_row_bytes;
    // copy-in: the kernel that last read buffer b (chunk i-2) must be done; for C as an
    // input, so must the copy-out that last read it
    if (i >= 2) {
      cudaStreamWaitEvent(c->pipe_in, c->ev_kernel[b], 0);
      if (p.c_is_input) cudaStreamWaitEvent(c->pipe_in, c->ev_out[b], 0);
    }
    if (!check_cuda(cudaMemcpyAsync(c->pipe_a[b], ha, (size_t)rows * p.a_row_bytes, cudaMemcpyHostToDevice, c->pipe_in),
                    "H2D chunk"))
      return false;
    if (p.c_is_input &&
        !check_cuda(cudaMemcpyAsync(c->pipe_c[b], hc, (size_t)rows * p.c_row_bytes, cudaMemcpyHostToDevice, c->pipe_in),
                    "H2D chunk"))
      return false;
    cudaEventRecord(c->ev_in[b], c->pipe_in);
    // kernel: needs its inputs, and the copy-out of chunk i-2 must have drained C buffer b
    cudaStreamWaitEvent(c->stream, c->ev_in[b], 0);
    if (i >= 2) cudaStreamWaitEvent(c->stream, c->ev_out[b], 0);
    if (!check_cuda(launch(rows, c->pipe_a[b], c->pipe_c[b]), "chunk kernel")) return false;
    cudaEventRecord(c->ev_kernel[b], c->stream);
    // copy-out
    if (i == 0) cudaStreamWaitEvent(c->pipe_out, c->ev_ready, 0);
    cudaStreamWaitEvent(c->pipe_out, c->ev_kernel[b], 0);
    if (!check_cuda(cudaMemcpyAsync(hc, c->pipe_c[b], (size_t)rows * p.c_row_bytes, cudaMemcpyDeviceToHost, c->pipe_out),
                    "D2H chunk"))
      return false;
    cudaEventRecord(c->ev_out[b], c->pipe_out);
  }
  if (!check_cuda(cudaStreamSynchronize(c->pipe_out), "cudaStreamSynchronize")) return false;
  if (!check_cuda(cudaStreamSynchronize(c->pipe_in), "cudaStreamSynchronize")) return false;
  return true;
}

}  // namespace exob200
