// One-shot all-reduce over peer memory for the split model's partial sums (no counterpart in the reference, which
// runs on one GPU).  Every rank's `output` / ffn `value` matmul writes its f32 partial [C, T] straight into a slot of
// the rank's exchange region, which the other ranks have mapped (CUDA IPC).  This kernel, one launch per rank:
//   1. tells every rank (itself included) that its slot is written: a system-scope release store of the call's
//      sequence number into that rank's flag word for this rank;
//   2. waits until all ranks' flags in its own region have reached the sequence number (local polls, bounded);
//   3. adds the slots of all ranks in rank order with plain 16-byte loads over NVLink, so every rank computes the
//      same sum bit for bit, and stores it rounded to the destination's dtype.
// Two slots alternate, so a rank may write its next partial while peers still read the previous one: a slot is
// written again only after the rank has passed the wait of the collective in between, which every peer reaches after
// its reads of that slot.  No TMA, no multicast, no library kernel touches peer memory.  A wait that gives up records
// WRK_ERR_TIMEOUT in the context's status word and the kernel runs on to its end (the sum is then meaningless).
#include <cuda_fp16.h>

#include <algorithm>

#include "device.cuh"
#include "kernels.h"

namespace wrk {
namespace k {

namespace {

constexpr uint32_t kPeerSpinLimit = 1u << 24;  // local polls of about 0.1 us: a couple of seconds

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_peer(const float4* p) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) peer_all_reduce_kernel(const PeerReduceArgs a) {
    __shared__ uint32_t s_seq;
    if (threadIdx.x == 0) s_seq = *a.epoch + 1;  // the same on every rank: all ranks run the same collectives in the same order
    __syncthreads();
    const uint32_t seq = s_seq;
    // this rank's slot was written by the kernel before this one on the stream
    if (blockIdx.x == 0 && threadIdx.x < a.world) {
        __threadfence_system();
        uint32_t* flags = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(a.regions[threadIdx.x]) + 2 * a.slot_bytes);
        st_release_sys(flags + a.rank, seq);
    }
    if (threadIdx.x < a.world) {
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(a.regions[a.rank]) + 2 * a.slot_bytes);
        bool ok = false;
        for (uint32_t i = 0; i < kPeerSpinLimit; ++i)
            if ((int32_t)(ld_acquire_sys(mine + threadIdx.x) - seq) >= 0) {
                ok = true;
                break;
            }
        if (!ok) atomicExch(a.status, (int32_t)WRK_ERR_TIMEOUT);
    }
    __syncthreads();
    const size_t vecs = a.count / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (size_t)gridDim.x * blockDim.x) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < a.world; ++r) {
            const float4 v = ld_peer(reinterpret_cast<const float4*>(static_cast<const uint8_t*>(a.regions[r]) + (size_t)a.slot * a.slot_bytes) + i);
            s.x += v.x;
            s.y += v.y;
            s.z += v.z;
            s.w += v.w;
        }
        if (a.dst_dtype == WRK_F16) {
            __half2* d = reinterpret_cast<__half2*>(a.dst) + 2 * i;
            d[0] = __floats2half2_rn(s.x, s.y);
            d[1] = __floats2half2_rn(s.z, s.w);
        } else {
            reinterpret_cast<float4*>(a.dst)[i] = s;
        }
    }
    // the last CTA to finish publishes the sequence number for the next call on this stream
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(a.done, 1u) == gridDim.x - 1) {
            *a.done = 0;
            *a.epoch = seq;
        }
    }
}

}  // namespace

cudaError_t peer_all_reduce(const PeerReduceArgs& a, int num_sms, cudaStream_t stream) {
    if (a.count == 0) return cudaSuccess;
    const size_t vecs = a.count / 4;
    const int grid = (int)std::min<size_t>((vecs + 255) / 256, (size_t)num_sms);
    peer_all_reduce_kernel<<<grid, 256, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace k
}  // namespace wrk
