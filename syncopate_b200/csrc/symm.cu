// Symmetric memory over CUDA IPC, flag barrier and status block: the replacement of the NVSHMEM
// runtime used by the reference's CommContext
// (syncopate/communication/comm_runtime/communication_context.py:31-106).
#include <errno.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "host_util.h"
#include "ptx.cuh"

struct syn_symm_record {
  void* local;
  void* peers[SYN_MAX_WORLD];
  size_t bytes;
};

struct syn_ctx {
  int rank, world, device;
  std::string dir;
  uint64_t seq;        // number of symmetric allocations so far (same on every rank)
  uint64_t barrier_epoch;
  std::vector<syn_symm_record> bufs;
  std::vector<std::string> my_files;
  int32_t* status;      // device int32[4]
  syn_symm barrier_flags;  // uint64[world] on every rank
};

namespace syn {

static void sleep_ms(int ms) {
  struct timespec ts = {ms / 1000, (ms % 1000) * 1000000L};
  nanosleep(&ts, nullptr);
}

static bool write_file_atomic(const std::string& path, const void* data, size_t n) {
  const std::string tmp = path + ".tmp";
  int fd = open(tmp.c_str(), O_CREAT | O_TRUNC | O_WRONLY, 0600);
  if (fd < 0) return false;
  const ssize_t w = write(fd, data, n);
  close(fd);
  if (w != static_cast<ssize_t>(n)) return false;
  return rename(tmp.c_str(), path.c_str()) == 0;
}

static bool read_file(const std::string& path, void* data, size_t n) {
  int fd = open(path.c_str(), O_RDONLY);
  if (fd < 0) return false;
  const ssize_t r = read(fd, data, n);
  close(fd);
  return r == static_cast<ssize_t>(n);
}

struct HandleRecord {
  cudaIpcMemHandle_t handle;
  uint64_t bytes;
};

__global__ void barrier_kernel(syn_symm flags, uint64_t epoch, uint64_t timeout_ns, int32_t* status) {
  __shared__ int abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  const int peer = threadIdx.x;
  if (peer < flags.world) {
    // everything this rank wrote before the barrier must be visible to a peer that sees the slot
    __threadfence_system();
    st_release_sys_u64(reinterpret_cast<uint64_t*>(flags.ptrs[peer]) + flags.rank, epoch);
    const uint64_t* mine = reinterpret_cast<const uint64_t*>(flags.ptrs[flags.rank]) + peer;
    if (!flag_wait_ge(mine, epoch, &abort_word, timeout_ns)) {
      if (status != nullptr && atomicCAS(status, 0, SYN_DEV_TIMEOUT_FLAG) == 0) {
        status[1] = -1;
        status[2] = peer;
        status[3] = -1;
      }
    }
  }
}

__global__ void flag_set_kernel(uint64_t* flag, uint64_t value) {
  __threadfence_system();
  st_release_sys_u64(flag, value);
}

__global__ void flag_wait_kernel(const uint64_t* flag, uint64_t value, uint64_t timeout_ns, int32_t* status,
                                 int tag) {
  __shared__ int abort_word;
  abort_word = 0;
  if (!flag_wait_ge(flag, value, &abort_word, timeout_ns)) {
    if (status != nullptr && atomicCAS(status, 0, SYN_DEV_TIMEOUT_FLAG) == 0) {
      status[1] = -1;
      status[2] = tag;
      status[3] = -1;
    }
  }
}

int preload_symm_kernels() {
  cudaFuncAttributes attr;
  SYN_CUDA_TRY(cudaFuncGetAttributes(&attr, barrier_kernel));
  SYN_CUDA_TRY(cudaFuncGetAttributes(&attr, flag_set_kernel));
  SYN_CUDA_TRY(cudaFuncGetAttributes(&attr, flag_wait_kernel));
  return SYN_OK;
}

}  // namespace syn

extern "C" {

int syn_preload(void) {
  using namespace syn;
  int rc = preload_symm_kernels();
  if (rc == SYN_OK) rc = preload_copy_kernels();
  if (rc == SYN_OK) rc = preload_fused_kernels();
  if (rc == SYN_OK) rc = preload_gemm_kernels();
  if (rc == SYN_OK) rc = preload_attn_kernels();
  if (rc == SYN_OK) SYN_CUDA_TRY(cudaDeviceSynchronize());
  return rc;
}

int syn_memcpy_async(void* dst, const void* src, size_t bytes, void* stream) {
  using namespace syn;
  if (dst == nullptr || src == nullptr) return SYN_ERR_INVALID;
  if (bytes == 0) return SYN_OK;
  SYN_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
  return SYN_OK;
}

int syn_flag_set(uint64_t* flag, uint64_t value, void* stream) {
  using namespace syn;
  if (flag == nullptr) return SYN_ERR_INVALID;
  // A stream memory operation needs no SM, so it cannot be starved by a persistent kernel that
  // fills the GPU while waiting for this very flag; the one-thread kernel is the fallback.
  typedef CUresult (*write_value_fn)(CUstream, CUdeviceptr, cuuint64_t, unsigned int);
  static write_value_fn write_value = nullptr;
  static bool looked_up = false;
  if (!looked_up) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue64", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      write_value = reinterpret_cast<write_value_fn>(fn);
    looked_up = true;
  }
  // (while the stream is being captured into a graph the kernel form is used: a kernel node is
  // always capturable)
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &capturing) != cudaSuccess) {
    cudaGetLastError();
    capturing = cudaStreamCaptureStatusNone;
  }
  if (write_value != nullptr && capturing == cudaStreamCaptureStatusNone) {
    CUresult r = write_value(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(flag), value, 0);
    if (r == CUDA_SUCCESS) return SYN_OK;
  }
  flag_set_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(flag, value);
  SYN_CUDA_TRY(cudaGetLastError());
  return SYN_OK;
}

int syn_flag_wait(const uint64_t* flag, uint64_t value, uint64_t timeout_ns, int32_t* status, int tag,
                  void* stream) {
  using namespace syn;
  if (flag == nullptr) return SYN_ERR_INVALID;
  flag_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      flag, value, timeout_ns ? timeout_ns : 2000000000ull, status, tag);
  SYN_CUDA_TRY(cudaGetLastError());
  return SYN_OK;
}

int syn_flag_wait_stream(const uint64_t* flag, uint64_t value, void* stream) {
  using namespace syn;
  if (flag == nullptr) return SYN_ERR_INVALID;
  typedef CUresult (*wait_value_fn)(CUstream, CUdeviceptr, cuuint64_t, unsigned int);
  static wait_value_fn wait_value = nullptr;
  static bool looked_up = false;
  if (!looked_up) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue64", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      wait_value = reinterpret_cast<wait_value_fn>(fn);
    looked_up = true;
  }
  if (wait_value == nullptr) return SYN_ERR_UNSUPPORTED;
  CUresult r = wait_value(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(flag), value,
                          CU_STREAM_WAIT_VALUE_GEQ);
  if (r != CUDA_SUCCESS) {
    char buf[64];
    snprintf(buf, sizeof(buf), "CUresult %d", static_cast<int>(r));
    set_cuda_error("cuStreamWaitValue64", buf);
    return SYN_ERR_CUDA;
  }
  return SYN_OK;
}

// Events that order a flag write on the flag stream behind a copy on a copy stream (timing off).
// A small ring per device: re-recording an event does not disturb waits already issued on it.
static cudaEvent_t ce_event(int dev) {
  constexpr int kRing = 256, kMaxDev = 64;
  static cudaEvent_t ring[kMaxDev][kRing];
  static unsigned next[kMaxDev];
  if (dev < 0 || dev >= kMaxDev) return nullptr;
  cudaEvent_t& e = ring[dev][next[dev]++ % kRing];
  if (e == nullptr && cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) e = nullptr;
  return e;
}

int syn_ce_run(const syn_ce_step* steps, int num_steps, void* const* streams, int num_streams, void* flag_stream,
               uint64_t value) {
  using namespace syn;
  if (steps == nullptr || num_steps < 0 || streams == nullptr || num_streams <= 0) return SYN_ERR_INVALID;
  int dev = 0;
  if (flag_stream != nullptr) SYN_CUDA_TRY(cudaGetDevice(&dev));
  for (int i = 0; i < num_steps; ++i) {
    const syn_ce_step& st = steps[i];
    if (st.stream < 0) return SYN_ERR_INVALID;
    void* sp = streams[st.stream % num_streams];
    int rc = SYN_OK;
    if (st.wait_flag != nullptr) rc = syn_flag_wait_stream(st.wait_flag, value, sp);
    if (rc == SYN_OK && st.bytes > 0) rc = syn_memcpy_async(st.dst, st.src, st.bytes, sp);
    if (rc == SYN_OK && st.set_flag != nullptr) {
      if (flag_stream != nullptr) {
        // the copy stream goes straight on to its next copy; the flag follows the copy through an event
        cudaEvent_t e = ce_event(dev);
        if (e == nullptr) return SYN_ERR_CUDA;
        SYN_CUDA_TRY(cudaEventRecord(e, static_cast<cudaStream_t>(sp)));
        SYN_CUDA_TRY(cudaStreamWaitEvent(static_cast<cudaStream_t>(flag_stream), e, 0));
        rc = syn_flag_set(st.set_flag, value, flag_stream);
      } else {
        rc = syn_flag_set(st.set_flag, value, sp);
      }
    }
    if (rc != SYN_OK) return rc;
  }
  return SYN_OK;
}

int syn_ctx_create(int rank, int world, int device, const char* rendezvous_dir, syn_ctx** out) {
  using namespace syn;
  if (out == nullptr || world <= 0 || world > SYN_MAX_WORLD || rank < 0 || rank >= world) return SYN_ERR_INVALID;
  if (world > 1 && (rendezvous_dir == nullptr || rendezvous_dir[0] == 0)) return SYN_ERR_INVALID;
  SYN_CUDA_TRY(cudaSetDevice(device));
  syn_ctx* c = new syn_ctx();
  c->rank = rank;
  c->world = world;
  c->device = device;
  c->dir = rendezvous_dir ? rendezvous_dir : "";
  c->seq = 0;
  c->barrier_epoch = 0;
  c->status = nullptr;
  if (world > 1) mkdir(c->dir.c_str(), 0700);  // may exist already
  cudaError_t e = cudaMalloc(&c->status, 4 * sizeof(int32_t));
  if (e == cudaSuccess) e = cudaMemset(c->status, 0, 4 * sizeof(int32_t));
  if (e != cudaSuccess) {
    set_cuda_error("cudaMalloc(status)", cudaGetErrorString(e));
    delete c;
    return SYN_ERR_CUDA;
  }
  int rc = syn_symm_alloc(c, sizeof(uint64_t) * SYN_MAX_WORLD, 0, &c->barrier_flags);
  // every kernel of the library is loaded now, while the GPU is idle: with lazy loading the first
  // launch of a kernel can wait for the kernels that are running, and a kernel that waits for a
  // peer must never be what such a launch waits for
  if (rc == SYN_OK) rc = syn_preload();
  if (rc != SYN_OK) {
    syn_ctx_destroy(c);
    return rc;
  }
  *out = c;
  return SYN_OK;
}

int syn_ctx_destroy(syn_ctx* c) {
  if (c == nullptr) return SYN_ERR_INVALID;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (auto& b : c->bufs) {
    for (int r = 0; r < c->world; ++r)
      if (r != c->rank && b.peers[r] != nullptr) cudaIpcCloseMemHandle(b.peers[r]);
    if (b.local != nullptr) cudaFree(b.local);
  }
  if (c->status != nullptr) cudaFree(c->status);
  for (auto& f : c->my_files) unlink(f.c_str());
  delete c;
  return SYN_OK;
}

int syn_symm_alloc(syn_ctx* c, size_t bytes, int timeout_s, syn_symm* out) {
  using namespace syn;
  if (c == nullptr || out == nullptr || bytes == 0) return SYN_ERR_INVALID;
  SYN_CUDA_TRY(cudaSetDevice(c->device));
  syn_symm_record rec;
  memset(&rec, 0, sizeof(rec));
  rec.bytes = bytes;
  SYN_CUDA_TRY(cudaMalloc(&rec.local, bytes));
  cudaError_t e = cudaMemset(rec.local, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_cuda_error("cudaMemset(symmetric buffer)", cudaGetErrorString(e));
    cudaFree(rec.local);
    return SYN_ERR_CUDA;
  }
  rec.peers[c->rank] = rec.local;
  const uint64_t seq = c->seq++;
  if (c->world > 1) {
    HandleRecord mine;
    memset(&mine, 0, sizeof(mine));
    e = cudaIpcGetMemHandle(&mine.handle, rec.local);
    if (e != cudaSuccess) {
      set_cuda_error("cudaIpcGetMemHandle", cudaGetErrorString(e));
      cudaFree(rec.local);
      return SYN_ERR_CUDA;
    }
    mine.bytes = bytes;
    char name[128];
    snprintf(name, sizeof(name), "/syn_%llu_%d.ipc", static_cast<unsigned long long>(seq), c->rank);
    const std::string my_path = c->dir + name;
    if (!write_file_atomic(my_path, &mine, sizeof(mine))) {
      cudaFree(rec.local);
      return SYN_ERR_RENDEZVOUS;
    }
    c->my_files.push_back(my_path);
    const int limit_ms = (timeout_s > 0 ? timeout_s : 120) * 1000;
    for (int r = 0; r < c->world; ++r) {
      if (r == c->rank) continue;
      snprintf(name, sizeof(name), "/syn_%llu_%d.ipc", static_cast<unsigned long long>(seq), r);
      const std::string path = c->dir + name;
      HandleRecord theirs;
      int waited = 0;
      while (!read_file(path, &theirs, sizeof(theirs))) {
        if (waited >= limit_ms) {
          c->bufs.push_back(rec);  // freed by syn_ctx_destroy
          return SYN_ERR_RENDEZVOUS;
        }
        sleep_ms(5);
        waited += 5;
      }
      if (theirs.bytes != bytes) {
        c->bufs.push_back(rec);
        return SYN_ERR_INVALID;  // ranks disagree on the allocation sequence
      }
      e = cudaIpcOpenMemHandle(&rec.peers[r], theirs.handle, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        set_cuda_error("cudaIpcOpenMemHandle", cudaGetErrorString(e));
        rec.peers[r] = nullptr;
        c->bufs.push_back(rec);
        return SYN_ERR_CUDA;
      }
    }
  }
  c->bufs.push_back(rec);
  out->world = c->world;
  out->rank = c->rank;
  for (int r = 0; r < SYN_MAX_WORLD; ++r) out->ptrs[r] = r < c->world ? rec.peers[r] : nullptr;
  return SYN_OK;
}

int syn_symm_free(syn_ctx* c, void* local_ptr) {
  if (c == nullptr || local_ptr == nullptr) return SYN_ERR_INVALID;
  for (size_t i = 0; i < c->bufs.size(); ++i) {
    if (c->bufs[i].local != local_ptr) continue;
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < c->world; ++r)
      if (r != c->rank && c->bufs[i].peers[r] != nullptr) cudaIpcCloseMemHandle(c->bufs[i].peers[r]);
    cudaFree(c->bufs[i].local);
    c->bufs.erase(c->bufs.begin() + i);
    return SYN_OK;
  }
  return SYN_ERR_INVALID;
}

int syn_barrier(syn_ctx* c, void* stream, uint64_t timeout_ns) {
  using namespace syn;
  if (c == nullptr) return SYN_ERR_INVALID;
  if (c->world == 1) return SYN_OK;
  const uint64_t epoch = ++c->barrier_epoch;
  barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      c->barrier_flags, epoch, timeout_ns ? timeout_ns : 2000000000ull, c->status);
  SYN_CUDA_TRY(cudaGetLastError());
  return SYN_OK;
}

int32_t* syn_ctx_status_ptr(syn_ctx* c) { return c ? c->status : nullptr; }

int syn_ctx_status(syn_ctx* c, void* stream, int32_t* out4) {
  using namespace syn;
  if (c == nullptr) return SYN_ERR_INVALID;
  SYN_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  int32_t host[4] = {0, 0, 0, 0};
  SYN_CUDA_TRY(cudaMemcpy(host, c->status, sizeof(host), cudaMemcpyDeviceToHost));
  if (out4 != nullptr) memcpy(out4, host, sizeof(host));
  if (host[0] != 0) SYN_CUDA_TRY(cudaMemset(c->status, 0, sizeof(host)));
  return status_to_err(host[0]);
}

}  // extern "C"
