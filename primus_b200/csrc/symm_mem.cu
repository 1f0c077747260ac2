// Symmetric-memory runtime: device allocations that every rank of a node-local group maps, plus the
// capability probe and the flag primitives the fused compute+collective kernels use.
//
//  * pb_symm_alloc / pb_symm_free: plain device allocations made outside the framework's caching
//    allocator, so that they can be exported.
//  * pb_ipc_export / pb_ipc_open / pb_ipc_close: CUDA IPC handle exchange (the handle bytes travel over the
//    process group's store / object collectives on the host side).
//  * pb_probe_p2p: peer-access matrix + capability bits.  Negative answers of optional-feature queries
//    leave a sticky error in the runtime; the probe clears it (cudaGetLastError) so that a failed
//    *optional* query never poisons the next kernel launch.  This is the job the reference's only
//    native source does with an LD_PRELOAD interposer on the HIP side
//    (runner/helpers/hooks/sdma/hip_attr_drain_preload.c:1-40,60-96,111-150); on CUDA no interposer is needed.
//  * pb_flag_*: tiny kernels that set / wait on 32-bit flags with release / acquire semantics at system
//    scope.  Waits are bounded: on expiry the kernel writes PB_ERR_TIMEOUT_FLAG to the status word and
//    returns, leaving the context usable.
//
// Replaces primus_turbo's symmetric-memory workspace (`get_symm_mem_workspace`,
// primus/backends/megatron/core/distributed/sdma_param_gather.py:39,189-196) and the ODC SHMEM shims
// (primus/core/odc/primitives/shmem_triton.py:130-463).
#include "common.cuh"

namespace {

__global__ void flag_set_kernel(int* flag, int value) { pb::set_flag_release(flag, value); }

__global__ void flag_wait_kernel(const int* flag, int value, int* status, long long max_cycles) {
  const long long t0 = clock64();
  int v;
  do {
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= value) return;
  } while (clock64() - t0 < max_cycles);
  atomicCAS(status, 0, PB_ERR_TIMEOUT_FLAG);
}

// Signals `value` into flags[my_rank] of every peer's flag array, then waits until every peer's
// signal arrived in the local array: a bounded device-side barrier over symmetric memory.
__global__ void symm_barrier_kernel(int* const* peer_flags, int* local_flags, int world, int my_rank, int value,
                                    int* status, long long max_cycles) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  pb::set_flag_release(peer_flags[r] + my_rank, value);
  const long long t0 = clock64();
  int v;
  do {
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(local_flags + r) : "memory");
    if (v >= value) return;
  } while (clock64() - t0 < max_cycles);
  atomicCAS(status, 0, PB_ERR_TIMEOUT_FLAG);
}

}  // namespace

extern "C" {

int pb_symm_alloc(void** out, long bytes) {
  cudaError_t e = cudaMalloc(out, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*out, 0, (size_t)bytes);
}
int pb_symm_free(void* p) { return (int)cudaFree(p); }

// handle_out: 64 bytes
int pb_ipc_export(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
int pb_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
int pb_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

// matrix_out: ndev*ndev ints (1 = device i can access device j). caps_out[0]: bit0 = all pairs have P2P,
// bit1 = multicast objects supported on the current device, bit2 = fabric handles supported.
int pb_probe_p2p(int* matrix_out, int max_dev, int* ndev_out, int* caps_out) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  if (n > max_dev) n = max_dev;
  *ndev_out = n;
  int all = 1;
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) {
      int can = (i == j);
      if (i != j && cudaDeviceCanAccessPeer(&can, i, j) != cudaSuccess) {
        cudaGetLastError();  // drain: an unsupported pair must not leave a sticky error behind
        can = 0;
      }
      matrix_out[i * max_dev + j] = can;
      if (!can) all = 0;
    }
  int caps = all ? 1 : 0;
  int dev = 0;
  cudaGetDevice(&dev);
  int v = 0;
  if (cudaDeviceGetAttribute(&v, (cudaDeviceAttr)132 /* cudaDevAttrMulticastSupported, optional */, dev) == cudaSuccess) {
    if (v) caps |= 2;
  } else {
    cudaGetLastError();
  }
  v = 0;
  if (cudaDeviceGetAttribute(&v, (cudaDeviceAttr)128 /* fabric handle support, optional */, dev) == cudaSuccess) {
    if (v) caps |= 4;
  } else {
    cudaGetLastError();
  }
  *caps_out = caps;
  return 0;
}

// One device-to-device copy on the GPU's copy engines (no SM work): `src` may be a peer's memory mapped into this
// process.  The parameter all-gather of the distributed optimizer issues one of these per peer and bucket on a side
// stream, which leaves every SM to the compute stream (the role of the reference's SDMA all-gather,
// primus/backends/megatron/core/distributed/sdma_param_gather.py).
int pb_copy_engine_pull(void* dst, const void* src, long bytes, cudaStream_t s) {
  if (bytes <= 0) return 0;
  return (int)cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, s);
}

int pb_flag_set(int* flag, int value, cudaStream_t s) {
  flag_set_kernel<<<1, 1, 0, s>>>(flag, value);
  return (int)cudaGetLastError();
}
int pb_flag_wait(const int* flag, int value, int* status, long max_cycles, cudaStream_t s) {
  flag_wait_kernel<<<1, 1, 0, s>>>(flag, value, status, max_cycles > 0 ? max_cycles : PB_WAIT_CYCLES);
  return (int)cudaGetLastError();
}
int pb_symm_barrier(int* const* peer_flags, int* local_flags, int world, int my_rank, int value, int* status,
                    long max_cycles, cudaStream_t s) {
  symm_barrier_kernel<<<1, 32, 0, s>>>(peer_flags, local_flags, world, my_rank, value, status,
                                        max_cycles > 0 ? max_cycles : PB_WAIT_CYCLES);
  return (int)cudaGetLastError();
}

}  // extern "C"
