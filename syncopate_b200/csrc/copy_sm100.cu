// syn_copy: a persistent SM copy kernel that executes a list of 2-D strided copies between
// peer-mapped buffers and raises a flag per copy - the stand-alone form of the comm warps, and the
// replacement of the reference's Triton persistent copy kernels
// (syncopate/communication/comm_runtime/tma_persistent_copy.py:114-171,
//  non_tma_persistent_copy.py:108-188) driven by SMCopyOp records.
#include "attn_sm100.cuh"
#include "host_util.h"

namespace syn {

constexpr int COPY_MAX_OPS = 64;
constexpr int COPY_THREADS = 512;

struct CopyParams {
  int32_t num_ops;
  uint32_t* counters;
  uint64_t signal_value;
  uint64_t timeout_ns;
  int32_t* status;
  CommOp ops[COPY_MAX_OPS];
  int8_t reduce[COPY_MAX_OPS];  // 0 = copy, 1 = dst += src as fp16, 2 = as bf16
};

// dst += v for eight 16-bit elements, as one vector reduction performed at the memory that owns
// `dst` (this GPU's or a peer's): concurrent reducing copies from several ranks into the same bytes
// do not lose updates.  Each addition rounds to the element type, as the reference's TMA reduce-add
// does (syncopate/communication/comm_runtime/tma_persistent_copy.py:129-169).
__device__ __forceinline__ void red_add16(void* dst, uint4 v, int kind) {
  if (kind == 2) {
    asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                 ::"l"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
  } else {
    asm volatile("red.relaxed.sys.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};"
                 ::"l"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
  }
}

__global__ void __launch_bounds__(COPY_THREADS) copy_kernel(const __grid_constant__ CopyParams p) {
  __shared__ int abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (int o = 0; o < p.num_ops; ++o) {
    const CommOp& op = p.ops[o];
    if (op.wait_flag != nullptr) {
      if (threadIdx.x == 0) flag_wait_ge(op.wait_flag, p.signal_value, &abort_word, p.timeout_ns);
      __syncthreads();
    }
    const size_t cpr = op.row_bytes / 16;  // 16-byte chunks per row
    const size_t total = cpr * op.rows;
    constexpr int U = 8;
    for (size_t i = tid; i < total; i += nthreads * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t j = i + u * nthreads;
        if (j < total) {
          const size_t r = j / cpr, c = j - r * cpr;
          v[u] = *reinterpret_cast<const uint4*>(op.src + r * op.src_pitch + c * 16);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t j = i + u * nthreads;
        if (j < total) {
          const size_t r = j / cpr, c = j - r * cpr;
          if (p.reduce[o] != 0) {
            red_add16(op.dst + r * op.dst_pitch + c * 16, v[u], p.reduce[o]);
          } else {
            *reinterpret_cast<uint4*>(op.dst + r * op.dst_pitch + c * 16) = v[u];
          }
        }
      }
    }
    if (op.set_flag != nullptr) {
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) {
        const uint32_t old = atomicAdd(&p.counters[o], 1u);
        if (old == gridDim.x - 1) {
          p.counters[o] = 0;
          __threadfence_system();
          st_release_sys_u64(op.set_flag, p.signal_value);
        }
      }
    }
  }
  if (threadIdx.x == 0 && abort_word != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0, abort_word) == 0) {
      p.status[1] = -1;
      p.status[2] = -1;
      p.status[3] = static_cast<int>(blockIdx.x);
    }
  }
}

int preload_copy_kernels() {
  cudaFuncAttributes attr;
  SYN_CUDA_TRY(cudaFuncGetAttributes(&attr, copy_kernel));
  return SYN_OK;
}

}  // namespace syn

extern "C" int syn_copy(const syn_attn_comm* comm, int num_sms, uint64_t signal_value, uint64_t timeout_ns,
                        int32_t* status, void* stream) {
  using namespace syn;
  if (comm == nullptr || comm->num_ops <= 0 || comm->ops == nullptr) return SYN_ERR_INVALID;
  if (comm->num_ops > COPY_MAX_OPS) return SYN_ERR_TOO_LARGE;
  if (comm->num_bufs <= 0 || comm->num_bufs > 4) return SYN_ERR_INVALID;
  CopyParams p;
  memset(&p, 0, sizeof(p));
  const int rank = comm->bufs[0].rank, world = comm->bufs[0].world;
  bool any_flag = false;
  for (int i = 0; i < comm->num_ops; ++i) {
    const syn_copy_op& o = comm->ops[i];
    if (o.src_buf < 0 || o.src_buf >= comm->num_bufs || o.dst_buf < 0 || o.dst_buf >= comm->num_bufs)
      return SYN_ERR_INVALID;
    if (o.src_rank < 0 || o.src_rank >= world || o.dst_rank < 0 || o.dst_rank >= world) return SYN_ERR_INVALID;
    if (o.src_rank != rank && o.dst_rank != rank) return SYN_ERR_INVALID;
    if ((o.src_offset | o.dst_offset | o.src_pitch | o.dst_pitch | o.row_bytes) & 15) return SYN_ERR_INVALID;
    CommOp& c = p.ops[i];
    const void* sb = comm->bufs[o.src_buf].ptrs[o.src_rank];
    void* db = comm->bufs[o.dst_buf].ptrs[o.dst_rank];
    if (sb == nullptr || db == nullptr) return SYN_ERR_INVALID;
    c.src = static_cast<const char*>(sb) + o.src_offset;
    c.dst = static_cast<char*>(db) + o.dst_offset;
    c.src_pitch = o.src_pitch;
    c.dst_pitch = o.dst_pitch;
    c.rows = o.rows;
    c.row_bytes = o.row_bytes;
    if (o.reduce != 0) {
      if (o.reduce != 1 || (o.dtype != SYN_DTYPE_F16 && o.dtype != SYN_DTYPE_BF16)) return SYN_ERR_UNSUPPORTED;
      p.reduce[i] = static_cast<int8_t>(o.dtype == SYN_DTYPE_BF16 ? 2 : 1);
    }
    if (o.flag >= 0) {
      if (o.flag_rank < 0 || o.flag_rank >= world || comm->flags.ptrs[o.flag_rank] == nullptr) return SYN_ERR_INVALID;
      c.set_flag = static_cast<uint64_t*>(comm->flags.ptrs[o.flag_rank]) + o.flag;
      any_flag = true;
    }
  }
  if (any_flag && comm->counters == nullptr) return SYN_ERR_INVALID;
  p.num_ops = comm->num_ops;
  p.counters = comm->counters;
  p.signal_value = signal_value ? signal_value : 1;
  p.timeout_ns = timeout_ns ? timeout_ns : 2000000000ull;
  p.status = status;
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != SYN_OK) return rc;
  const int grid = num_sms > 0 ? (num_sms < sms ? num_sms : sms) : sms;
  copy_kernel<<<grid, COPY_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(p);
  SYN_CUDA_TRY(cudaGetLastError());
  return SYN_OK;
}
