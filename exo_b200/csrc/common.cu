// Context management, thread-local error state and host<->device staging.
#include "common.cuh"
#include "kernels.cuh"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

namespace exob200 {

namespace {
thread_local int tl_code = EXO_B200_OK;
thread_local std::string tl_msg;
std::mutex g_mutex;
std::map<int, exo_b200_Context*> g_default;  // one default context per device
thread_local cudaStream_t tl_default_stream = nullptr;
}  // namespace

void set_error(int code, const std::string& msg) {
  tl_code = code;
  tl_msg = msg;
  if (getenv("EXOB200_VERBOSE")) fprintf(stderr, "[exo_b200] error %d: %s\n", code, msg.c_str());
}
void clear_error() {
  tl_code = EXO_B200_OK;
  tl_msg.clear();
}
int last_error_code() { return tl_code; }
const char* last_error_msg() { return tl_msg.c_str(); }

bool check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return true;
  set_error(EXO_B200_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
  return false;
}

static exo_b200_Context* make_context(int device, cudaStream_t stream) {
  cudaDeviceProp prop;
  if (!check_cuda(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties")) return nullptr;
  if (prop.major != 10) {
    set_error(EXO_B200_ERR_UNSUPPORTED,
              std::string("device '") + prop.name + "' is sm_" + std::to_string(prop.major) +
                  std::to_string(prop.minor) + "; this library contains sm_100a code only");
    return nullptr;
  }
  exo_b200_Context* c = new exo_b200_Context();
  memset(c, 0, sizeof(*c));
  c->magic = kContextMagic;
  c->device = device;
  c->stream = stream;
  c->sm_count = prop.multiProcessorCount;
  c->sgemm_path = EXO_B200_SGEMM_FFMA;
  c->mutex = new std::recursive_mutex();
  if (const char* p = getenv("EXOB200_SGEMM_PATH")) {
    if (!strcmp(p, "3xtf32")) c->sgemm_path = EXO_B200_SGEMM_3XTF32;
  }
  int cur = 0;
  cudaGetDevice(&cur);
  cudaSetDevice(device);
  void* host = nullptr;
  cudaError_t e = cudaHostAlloc(&host, sizeof(DeviceStatus), cudaHostAllocMapped);
  if (e == cudaSuccess) {
    memset(host, 0, sizeof(DeviceStatus));
    c->status_host = static_cast<DeviceStatus*>(host);
    void* dev = nullptr;
    e = cudaHostGetDevicePointer(&dev, host, 0);
    c->status_dev = static_cast<DeviceStatus*>(dev);
  }
  cudaSetDevice(cur);
  if (!check_cuda(e, "status word allocation")) {
    delete c->mutex;
    delete c;
    return nullptr;
  }
  return c;
}

exo_b200_Context* default_context() {
  int device = 0;
  if (!check_cuda(cudaGetDevice(&device), "cudaGetDevice")) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_default.find(device);
  if (it == g_default.end()) {
    exo_b200_Context* c = make_context(device, nullptr);
    if (!c) return nullptr;
    c->is_default = true;
    it = g_default.emplace(device, c).first;
  }
  return it->second;
}

// A context belongs to one device: its stream, staging, scratch and SM count are that
// device's.  If another device is current when an entry point is called, the context's
// device is made current for the length of the call and the caller's choice restored
// afterwards; if that fails the call is refused (get() returns nullptr, error set).
ContextUse::ContextUse(exo_b200_Context* c) : c_(c), restore_device_(-1) {
  if (!c_) return;
  c_->mutex->lock();
  if (c_->is_default) c_->stream = tl_default_stream;
  int cur = -1;
  if (cudaGetDevice(&cur) == cudaSuccess && cur != c_->device) {
    if (!check_cuda(cudaSetDevice(c_->device), "cudaSetDevice(context's device)")) {
      c_->mutex->unlock();
      c_ = nullptr;
      return;
    }
    restore_device_ = cur;
  }
}
ContextUse::~ContextUse() {
  if (!c_) return;
  if (restore_device_ >= 0) cudaSetDevice(restore_device_);
  c_->mutex->unlock();
}

exo_b200_Context* resolve_context(void* ctxt) {
  if (ctxt == nullptr) return default_context();
  exo_b200_Context* c = static_cast<exo_b200_Context*>(ctxt);
  if (c->magic != kContextMagic) {
    set_error(EXO_B200_ERR_INVALID_ARGUMENT, "ctxt is neither NULL nor an exo_b200_Context");
    return nullptr;
  }
  return c;
}

bool is_device_pointer(const void* p) {
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, p);
  if (e != cudaSuccess) {
    cudaGetLastError();  // unregistered host memory on old drivers: clear and treat as host
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

int owning_device(const void* p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return attr.type == cudaMemoryTypeDevice ? attr.device : -1;
}

bool stage_in(exo_b200_Context* c, int slot, const void* user, size_t bytes, bool copy_in, Operand* op) {
  op->user = user;
  op->bytes = bytes;
  cudaPointerAttributes attr;
  bool on_device = false;
  if (cudaPointerGetAttributes(&attr, user) == cudaSuccess) {
    on_device = attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
    if (attr.type == cudaMemoryTypeDevice && attr.device != c->device) {
      // the kernels run on the context's device and would dereference memory of another GPU
      set_error(EXO_B200_ERR_INVALID_ARGUMENT,
                "a device pointer belongs to device " + std::to_string(attr.device) + " but the context is on device " +
                    std::to_string(c->device));
      return false;
    }
  } else {
    cudaGetLastError();  // unregistered host memory on old drivers: clear and treat as host
  }
  if (on_device) {
    op->dev = const_cast<void*>(user);
    op->staged = false;
    return true;
  }
  if (c->stage_bytes[slot] < bytes) {
    if (c->stage[slot]) {
      if (!check_cuda(cudaStreamSynchronize(c->stream), "cudaStreamSynchronize")) return false;
      cudaFree(c->stage[slot]);
      c->stage[slot] = nullptr;
      c->stage_bytes[slot] = 0;
    }
    size_t want = bytes + bytes / 8 + 256;
    if (!check_cuda(cudaMalloc(&c->stage[slot], want), "cudaMalloc(staging)")) return false;
    c->stage_bytes[slot] = want;
  }
  op->dev = c->stage[slot];
  op->staged = true;
  if (copy_in &&
      !check_cuda(cudaMemcpyAsync(op->dev, user, bytes, cudaMemcpyHostToDevice, c->stream), "H2D copy"))
    return false;
  return true;
}

bool stage_out(exo_b200_Context* c, const Operand& op) {
  if (!op.staged) return true;
  return check_cuda(cudaMemcpyAsync(const_cast<void*>(op.user), op.dev, op.bytes, cudaMemcpyDeviceToHost,
                                    c->stream),
                    "D2H copy");
}

static bool read_status(exo_b200_Context* c) {
  if (c->status_host && c->status_host->code != 0) {
    DeviceStatus s = *c->status_host;
    memset(c->status_host, 0, sizeof(DeviceStatus));
    char buf[160];
    snprintf(buf, sizeof(buf), "device-side wait ran out (kernel location %d, block %d, detail %d)",
             s.where, s.block, s.detail);
    set_error(s.code, buf);
    return false;
  }
  return true;
}

bool finish(exo_b200_Context* c, bool any_staged) {
  if (!any_staged) return true;
  if (!check_cuda(cudaStreamSynchronize(c->stream), "cudaStreamSynchronize")) return false;
  return read_status(c);
}

static bool pipeline_streams(exo_b200_Context* c) {
  if (c->pipe_ready) return true;
  if (!check_cuda(cudaStreamCreateWithFlags(&c->pipe_in, cudaStreamNonBlocking), "cudaStreamCreate")) return false;
  if (!check_cuda(cudaStreamCreateWithFlags(&c->pipe_out, cudaStreamNonBlocking), "cudaStreamCreate")) return false;
  for (int i = 0; i < 2; i++) {
    cudaEventCreateWithFlags(&c->ev_in[i], cudaEventDisableTiming);
    cudaEventCreateWithFlags(&c->ev_kernel[i], cudaEventDisableTiming);
    cudaEventCreateWithFlags(&c->ev_out[i], cudaEventDisableTiming);
  }
  if (!check_cuda(cudaEventCreateWithFlags(&c->ev_ready, cudaEventDisableTiming), "cudaEventCreate")) return false;
  c->pipe_ready = true;
  return true;
}

bool pipeline_prepare(exo_b200_Context* c, size_t a_chunk_bytes, size_t c_chunk_bytes) {
  if (!pipeline_streams(c)) return false;
  if (c->pipe_a_bytes < a_chunk_bytes || c->pipe_c_bytes < c_chunk_bytes) {
    if (!check_cuda(cudaStreamSynchronize(c->stream), "cudaStreamSynchronize")) return false;
    for (int i = 0; i < 2; i++) {
      if (c->pipe_a[i]) cudaFree(c->pipe_a[i]);
      if (c->pipe_c[i]) cudaFree(c->pipe_c[i]);
      c->pipe_a[i] = c->pipe_c[i] = nullptr;
    }
    c->pipe_a_bytes = c->pipe_c_bytes = 0;
    for (int i = 0; i < 2; i++) {
      if (!check_cuda(cudaMalloc(&c->pipe_a[i], a_chunk_bytes), "cudaMalloc(pipeline)")) return false;
      if (!check_cuda(cudaMalloc(&c->pipe_c[i], c_chunk_bytes), "cudaMalloc(pipeline)")) return false;
    }
    c->pipe_a_bytes = a_chunk_bytes;
    c->pipe_c_bytes = c_chunk_bytes;
  }
  return true;
}

static bool ensure_stage(exo_b200_Context* c, int slot, size_t bytes) {
  if (c->stage_bytes[slot] >= bytes) return true;
  if (c->stage[slot]) {
    if (!check_cuda(cudaStreamSynchronize(c->stream), "cudaStreamSynchronize")) return false;
    cudaFree(c->stage[slot]);
    c->stage[slot] = nullptr;
    c->stage_bytes[slot] = 0;
  }
  const size_t want = bytes + bytes / 8 + 256;
  if (!check_cuda(cudaMalloc(&c->stage[slot], want), "cudaMalloc(staging)")) return false;
  c->stage_bytes[slot] = want;
  return true;
}

bool block_pipeline_prepare(exo_b200_Context* c, size_t a_bytes, size_t b_bytes, size_t c_block_bytes) {
  if (!pipeline_streams(c)) return false;
  if (!c->blk_ready) {
    for (int i = 0; i < 4; i++) {
      cudaEventCreateWithFlags(&c->ev_blk_kernel[i], cudaEventDisableTiming);
      cudaEventCreateWithFlags(&c->ev_blk_out[i], cudaEventDisableTiming);
    }
    if (!check_cuda(cudaEventCreateWithFlags(&c->ev_upload, cudaEventDisableTiming), "cudaEventCreate")) return false;
    c->blk_ready = true;
  }
  if (!ensure_stage(c, 0, a_bytes) || !ensure_stage(c, 1, b_bytes)) return false;
  if (c->blk_c_bytes < c_block_bytes) {
    if (!check_cuda(cudaStreamSynchronize(c->stream), "cudaStreamSynchronize")) return false;
    for (int i = 0; i < 4; i++) {
      if (c->blk_c[i]) cudaFree(c->blk_c[i]);
      c->blk_c[i] = nullptr;
    }
    c->blk_c_bytes = 0;
    for (int i = 0; i < 4; i++)
      if (!check_cuda(cudaMalloc(&c->blk_c[i], c_block_bytes), "cudaMalloc(block pipeline)")) return false;
    c->blk_c_bytes = c_block_bytes;
  }
  return true;
}

std::vector<char> block_upload_order(const BlockPipeline& p) {
  const int64_t na = (p.rows + p.chunk_rows - 1) / p.chunk_rows, nb = (p.cols + p.chunk_cols - 1) / p.chunk_cols;
  std::vector<char> order;
  order.reserve((size_t)(na + nb));
  int64_t a = 0, b = 0;
  while (a < na || b < nb) {
    // output bytes enabled per input byte: a row chunk enables b blocks, a column block a blocks
    const double gain_a = a < na ? (double)b * p.chunk_cols * p.c_elem_bytes / (double)p.a_row_bytes : -1.0;
    const double gain_b = b < nb ? (double)a * p.chunk_rows * p.c_elem_bytes / (double)p.b_col_bytes : -1.0;
    if (gain_a >= gain_b) {
      order.push_back('A');
      a++;
    } else {
      order.push_back('B');
      b++;
    }
  }
  return order;
}

static bool stream_is_capturing(cudaStream_t s) {
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &cap) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return cap != cudaStreamCaptureStatusNone;
}

bool acquire_scratch(exo_b200_Context* c, int slot, size_t bytes) {
  if (!ensure_scratch(c, slot, bytes)) return false;
  if (c->scratch_busy[slot] && c->scratch_stream[slot] != c->stream) {
    // A stream that is being captured may not depend on work outside its capture; a caller who
    // captures orders the captured graph against earlier uses of the context themselves.
    if (stream_is_capturing(c->stream)) return true;
    // cudaStreamWaitEvent on an event that has completed costs nothing on the device
    if (!check_cuda(cudaStreamWaitEvent(c->stream, c->scratch_ev[slot], 0), "cudaStreamWaitEvent(scratch)"))
      return false;
  }
  return true;
}

void release_scratch(exo_b200_Context* c, int slot) {
  // An event recorded while the stream is being captured belongs to the capture and cannot be
  // waited on from outside it; a capturing caller orders its own streams.
  if (stream_is_capturing(c->stream)) return;
  if (!c->scratch_ev[slot] &&
      cudaEventCreateWithFlags(&c->scratch_ev[slot], cudaEventDisableTiming) != cudaSuccess) {
    cudaGetLastError();
    c->scratch_ev[slot] = nullptr;
    return;
  }
  if (cudaEventRecord(c->scratch_ev[slot], c->stream) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  c->scratch_stream[slot] = c->stream;
  c->scratch_busy[slot] = true;
}

bool ensure_scratch(exo_b200_Context* c, int slot, size_t bytes) {
  if (c->scratch_bytes[slot] >= bytes) return true;
  if (c->scratch[slot]) {
    // cudaFree waits for all work on the device, other streams' readers of the slot included
    if (!check_cuda(cudaStreamSynchronize(c->stream), "cudaStreamSynchronize")) return false;
    cudaFree(c->scratch[slot]);
    c->scratch[slot] = nullptr;
    c->scratch_bytes[slot] = 0;
    if (slot == 2) c->wkey_valid = false;
  }
  if (!check_cuda(cudaMalloc(&c->scratch[slot], bytes), "cudaMalloc(scratch)")) return false;
  c->scratch_bytes[slot] = bytes;
  return true;
}

}  // namespace exob200

using namespace exob200;

extern "C" {

exo_b200_Context* exo_b200_context_create(int device, void* stream) {
  clear_error();
  if (device < 0 && !check_cuda(cudaGetDevice(&device), "cudaGetDevice")) return nullptr;
  return make_context(device, static_cast<cudaStream_t>(stream));
}

void exo_b200_context_destroy(exo_b200_Context* c) {
  if (!c || c->magic != kContextMagic) return;
  c->mutex->lock();  // waits for a call in flight on another thread
  int cur = -1;
  cudaGetDevice(&cur);
  if (cur != c->device) cudaSetDevice(c->device);  // streams, events and allocations are this device's
  cudaStreamSynchronize(c->stream);
  for (int i = 0; i < 4; i++)
    if (c->stage[i]) cudaFree(c->stage[i]);
  for (int i = 0; i < 3; i++) {
    if (c->scratch[i]) cudaFree(c->scratch[i]);
    if (c->scratch_ev[i]) cudaEventDestroy(c->scratch_ev[i]);
  }
  if (c->status_host) cudaFreeHost(c->status_host);
  if (c->pipe_ready) {
    cudaStreamDestroy(c->pipe_in);
    cudaStreamDestroy(c->pipe_out);
    for (int i = 0; i < 2; i++) {
      cudaEventDestroy(c->ev_in[i]);
      cudaEventDestroy(c->ev_kernel[i]);
      cudaEventDestroy(c->ev_out[i]);
      if (c->pipe_a[i]) cudaFree(c->pipe_a[i]);
      if (c->pipe_c[i]) cudaFree(c->pipe_c[i]);
    }
    cudaEventDestroy(c->ev_ready);
  }
  if (c->blk_ready) {
    for (int i = 0; i < 4; i++) {
      cudaEventDestroy(c->ev_blk_kernel[i]);
      cudaEventDestroy(c->ev_blk_out[i]);
    }
    cudaEventDestroy(c->ev_upload);
  }
  for (int i = 0; i < 4; i++)
    if (c->blk_c[i]) cudaFree(c->blk_c[i]);
  c->magic = 0;
  if (cur >= 0 && cur != c->device) cudaSetDevice(cur);
  c->mutex->unlock();
  delete c->mutex;
  delete c;
}

void exo_b200_context_set_stream(exo_b200_Context* c, void* stream) {
  if (!c || c->magic != kContextMagic) return;
  ContextUse use(c);
  c->stream = static_cast<cudaStream_t>(stream);
}

void exo_b200_context_set_sgemm_path(exo_b200_Context* c, int path) {
  if (!c || c->magic != kContextMagic) return;
  ContextUse use(c);
  c->sgemm_path = path;
}

void exo_b200_context_cache_weights(exo_b200_Context* ctxt, int enable) {
  clear_error();
  ContextUse use(resolve_context(ctxt));
  exo_b200_Context* c = use.get();
  if (!c) return;
  c->cache_weights = enable != 0;
  c->wkey_valid = false;
}

void exo_b200_context_invalidate(exo_b200_Context* ctxt) {
  clear_error();
  ContextUse use(resolve_context(ctxt));
  exo_b200_Context* c = use.get();
  if (c) c->wkey_valid = false;
}

void exo_b200_set_default_stream(void* stream) { tl_default_stream = static_cast<cudaStream_t>(stream); }

int exo_b200_synchronize(exo_b200_Context* ctxt) {
  clear_error();
  ContextUse use(resolve_context(ctxt));
  exo_b200_Context* c = use.get();
  if (!c) return exo_b200_last_error();
  if (check_cuda(cudaStreamSynchronize(c->stream), "cudaStreamSynchronize") && read_status(c))
    collect_static_status();
  return exo_b200_last_error();
}

int exo_b200_last_error(void) { return last_error_code(); }
const char* exo_b200_last_error_string(void) { return last_error_msg(); }
const char* exo_b200_version(void) { return "exo_b200 0.1 (sm_100a)"; }

}  // extern "C"
