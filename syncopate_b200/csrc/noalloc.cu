// syn_gemm_noalloc: the flag-raising (producer) GEMM for hosts that must not allocate.
//
// The producer GEMM counts the finished tiles of every wave in a small scratch array and raises
// the wave's flag when the count is complete.  syn_gemm takes that array from the caller.  Some
// callers have nowhere to get it from: a serving process that has handed the whole GPU to its own
// memory pool at start-up, a step function that runs where a device-synchronising cudaMalloc is
// forbidden (latency-critical loops, regions replayed from a recorded launch sequence), or a
// plugin loaded into a host that forbids allocation after initialisation.  For them the scratch
// lives in this library's image instead: a file-scope device array, one copy per GPU that loads the
// library, held until the process exits.
#include <atomic>

#include "gemm_host.h"

namespace {

// SYN_MAX_WAVES counters of 4 bytes = 256 bytes per GPU.
__device__ __align__(256) uint32_t g_wave_counters[SYN_MAX_WAVES];

constexpr int kMaxDevices = 64;
// device address of g_wave_counters, per device, null = not looked up yet (two host threads that
// look it up at the same time store the same value)
std::atomic<uint32_t*> g_counters_addr[kMaxDevices];

}  // namespace

extern "C" int syn_gemm_noalloc(const syn_gemm_args* args, const syn_schedule* sched,
                                const syn_schedule* producer_sched, void* stream) {
  using namespace syn;
  if (args == nullptr || producer_sched == nullptr) return SYN_ERR_INVALID;
  if (producer_sched->num_waves <= 0) return SYN_ERR_INVALID;
  if (producer_sched->num_waves > SYN_MAX_WAVES) return SYN_ERR_TOO_LARGE;  // scratch holds SYN_MAX_WAVES counters
  if (sched != nullptr && sched->num_waves > SYN_MAX_WAVES) return SYN_ERR_TOO_LARGE;
  int dev = -1;
  SYN_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return SYN_ERR_UNSUPPORTED;
  if (g_counters_addr[dev].load(std::memory_order_acquire) == nullptr) {
    // In host code the array's name is only a handle; the address kernels can use has to be asked
    // for, once per device, with that device current.
    void* p = nullptr;
    SYN_CUDA_TRY(cudaGetSymbolAddress(&p, g_wave_counters));
    if (p == nullptr) return SYN_ERR_CUDA;
    g_counters_addr[dev].store(static_cast<uint32_t*>(p), std::memory_order_release);
  }
  uint32_t* counters = g_counters_addr[dev].load(std::memory_order_acquire);
  // Every call shares the array and it keeps what the last call left: a call that ended in a
  // timeout may leave partial counts behind, so start from zero each time (stream-ordered).
  SYN_CUDA_TRY(cudaMemsetAsync(counters, 0, sizeof(uint32_t) * SYN_MAX_WAVES, static_cast<cudaStream_t>(stream)));
  syn_gemm_args local = *args;
  local.producer_counter_ptr = counters;
  return syn_gemm(&local, sched, producer_sched, stream);
}
