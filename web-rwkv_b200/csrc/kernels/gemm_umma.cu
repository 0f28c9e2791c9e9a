// Tensor-memory GEMM for the prefill / batched path (matmul_mat_fp16 / int8 / nf4 with 16 or more tokens):
// out[n][m] = act(sum_k W[m][k] * x[n][k]).
//
// One CTA owns a 128-row slice of W and up to 256 tokens and walks K in steps of 64.  Warp roles:
//   * warp 9 (one lane) streams the packed weight tiles with TMA (cp.async.bulk.tensor.2d): 128 rows x 64
//     (Int8) or 32 (NF4) bytes per step into a ring of raw stages several steps ahead of their use; fp16
//     weights go straight into the A operand stage through a 128-byte-swizzled tensor map;
//   * warp 10 (one lane) streams the fp16 activations of the step, [tokens x 64] through a 128-byte-swizzled
//     tensor map, into the B operand stage (rows past the last token are zero-filled by the TMA unit);
//   * warps 0-7 dequantize as two groups of four warps on alternate pairs of steps: a thread turns the 64
//     weights of one row and step into fp16 (f32 math, one rounding) and stores them in the K-major
//     128-byte-swizzled layout tcgen05 reads; the (min, max) / absmax values of the next 256 columns are
//     fetched with cp.async while the current ones are in use;
//   * warp 8 (one lane) issues tcgen05.mma.cta_group::1.kind::f16 (M = 128, N = token tile, K = 16, four per
//     step) into a TMEM accumulator of 128 lanes x N fp32 columns and releases the stage with tcgen05.commit;
//   * after the last step warps 0-7 read the accumulator back with tcgen05.ld (warp w reads lanes
//     32 (w % 4) ..), apply the activation and put the tile, in the output's type, into shared memory (the operand
//     stages are free by then), from where it goes to global memory in 16-byte pieces: the 128 rows of a token are
//     adjacent elements of the output.
// A launch takes up to four matrices of one format, K and token count (UmmaGroup): their row tiles share grid.x, so
// key / value / receptance / gate of a layer fill the SMs together and none has to split K.
// At 256 tokens the K walk is paced by the L2: every CTA re-reads the whole [tokens x K] activation tile next to its
// own 128 rows of weights (40 KB per step and CTA; four 4096 x 4096 matrices at 256 tokens: 335 MB in 43 us, 7.7 TB/s),
// which neither fewer dequantizing instructions (packed add.f32x2 / fma.rn.f32x2) nor a fourth operand stage change much.
// Where the output tiles alone leave SMs idle, the CTAs of a thread-block cluster (up to 8, along grid.z) split the
// K range of one tile: each writes its partial accumulator to its own shared memory and, after a cluster barrier,
// adds its share of the columns over all peers through distributed shared memory.
// Weights enter the MMA as fp16(fma(q, (max - min) / 255, min)) resp. fp16(table[nib] * absmax), computed in
// f32 and rounded once; the accumulation is fp32.  Every wait on an mbarrier is bounded: on a timeout the
// kernel records WRK_ERR_TIMEOUT in the context's status word, stops waiting and still frees its TMEM.
#include <cuda.h>

#include "device.cuh"
#include "kernels.h"

namespace wrk {
namespace k {

namespace {

constexpr int BM = 128;             // weight rows per CTA (UMMA M)
constexpr int BK = 64;              // K per stage: one 128-byte swizzle atom of fp16
constexpr int kDequantWarps = 8;
constexpr int kMmaWarp = 8, kWeightTmaWarp = 9;  // warp 10 streams the activations
constexpr int kUmmaThreads = 11 * 32;
constexpr int kMaxStages = 6;       // operand stages
constexpr int kMaxRaw = 8;          // raw weight stages
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr uint32_t A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr uint32_t SCALE_SLOT_BYTES = BM * 8;    // 8 bytes of scales per row and 256 columns

struct UmmaParams {
    const uint8_t* w;
    const __half* scale;
    const float* table;
    int kind;
    uint32_t K, M, N;
    DView out;
    int act;
    uint32_t n_tile;    // tokens per CTA: multiple of 16, <= 256
    uint32_t tmem_cols; // power of two >= max(32, n_tile)
    uint32_t stages;    // operand stages
    uint32_t raw;       // raw weight stages (quantized kinds)
    uint32_t splits;    // CTAs along K per output tile (grid.z = the cluster's size)
    int32_t* status;
};

// Up to kMaxGroup problems of one weight format, K, token count and tiling in one launch: the row tiles of problem i
// are CTAs tile_start[i] .. tile_start[i + 1] - 1 along grid.x.  Matrices that read different activations at the same
// point of a layer (key / value / receptance / gate) fill the SMs together, where each alone would have to split K
// and pay for the exchange of partial tiles.
constexpr int kMaxGroup = 4;
struct alignas(64) UmmaGroup {
    CUtensorMap map_w[kMaxGroup], map_x[kMaxGroup];
    UmmaParams p[kMaxGroup];
    uint32_t tile_start[kMaxGroup + 1];
    uint32_t count;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// 2-D tiled TMA load of the box at (x, y) into this CTA's shared memory at dst, completing on bar.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(
                     smem_addr(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_addr(bar)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void cp_async8z(void* dst, const void* src, bool valid) {
    const uint32_t n = valid ? 8u : 0u;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(n) : "memory");
}
// Waits for the phase with the given parity; gives up after kSpinLimit polls (or at once when another
// wait of this CTA has already given up) and reports it.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int32_t* status) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(ok)
            : "r"(smem_addr(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    if (status != nullptr) atomicExch(status, (int32_t)WRK_ERR_TIMEOUT);
    return false;
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// K-major, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart, 16-byte chunk index XOR row % 8.
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk) {
    return (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4);
}
// Shared-memory matrix descriptor of such a tile (start address, LBO = 1, SBO = 1024 bytes, version 1, SWIZZLE_128B).
__device__ __forceinline__ uint64_t sw128_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor: fp16 x fp16 -> fp32, both operands K-major, M x N.
__device__ __forceinline__ uint32_t f16_idesc(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t v[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Thread-block cluster: hardware barrier over all threads of all CTAs of the cluster, and 16-byte loads from
// a peer CTA's shared memory.
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ float4 ld_peer_smem(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local_addr), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(remote)
                 : "memory");
    return v;
}

__device__ __forceinline__ uint32_t pack_half2(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

// Two variations measured the same as this arrangement and were dropped: sixteen dequantizing warps, each taking half of
// a step's columns (Int8 4096 x 4096 at 64 / 1024 tokens: 19.3 / 72.5 us against 19.1 / 74.4 us), and four MMA issuer
// warps with an accumulator each (19.2 us at 64 tokens, slower at 256).  Neither the convert chain's latency nor the
// single issuing thread paces the kernel at few tokens; its fixed work per launch does (set-up, pipeline fill,
// epilogue, cluster reduction: about 10 of the 19 us).
// 32 (Int8) weights of one row, raw bytes in `q0, q1`, block scale (min, max) -> four 16-byte groups of fp16.
__device__ __forceinline__ void dequant_int8(uint4 q0, uint4 q1, uint32_t minmax, uint4 out[4]) {
    // f32 dequantization, one rounding to fp16 per weight: the errors of a row are independent, none is
    // shared by a whole block
    const float2 mm = __half22float2(*reinterpret_cast<const __half2*>(&minmax));
    const float sc = (mm.y - mm.x) * (1.0f / 255.0f), mn = mm.x;
    const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    const float2 sc2 = make_float2(sc, sc), mn2 = make_float2(mn, mn), bias2 = make_float2(-8388608.0f, -8388608.0f);
    uint32_t h[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        // byte b -> float 8388608 + b (0x4B000000 | b), minus 8388608: b exactly; two weights per instruction from
        // there on (add.f32x2, fma.rn.f32x2: the same roundings as the scalar forms)
        const float2 f01 = make_float2(__uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7650)),
                                       __uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7651)));
        const float2 f23 = make_float2(__uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7652)),
                                       __uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7653)));
        h[2 * i] = pack_half2(__float22half2_rn(__ffma2_rn(__fadd2_rn(f01, bias2), sc2, mn2)));
        h[2 * i + 1] = pack_half2(__float22half2_rn(__ffma2_rn(__fadd2_rn(f23, bias2), sc2, mn2)));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) out[j] = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
}
// 32 NF4 weights (16 bytes, low nibble first) of one 64-weight block with absmax `am`.
__device__ __forceinline__ void dequant_nf4(uint4 q, float am, const float2* lut2, uint4 out[4]) {
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
    uint32_t h[16];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float2 pair = lut2[(words[i] >> (8 * b)) & 0xffu];  // (table[lo nibble], table[hi nibble])
            h[4 * i + b] = pack_half2(__float22half2_rn(__fmul2_rn(pair, make_float2(am, am))));
        }
#pragma unroll
    for (int j = 0; j < 4; ++j) out[j] = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
}

// One instantiation per weight format: the dequantizing loop holds only its own format's code.
template <int KIND>
__global__ void __launch_bounds__(kUmmaThreads, 1)
matmul_umma_kernel(const __grid_constant__ UmmaGroup grp) {
    extern __shared__ uint8_t smem_raw[];
    uint32_t gi = 0;
#pragma unroll
    for (uint32_t i = 1; i < (uint32_t)kMaxGroup; ++i)
        if (i < grp.count && blockIdx.x >= grp.tile_start[i]) gi = i;
    const UmmaParams& p = grp.p[gi];
    const CUtensorMap& map_w = grp.map_w[gi];
    const CUtensorMap& map_x = grp.map_x[gi];
    __shared__ uint64_t ab_full[kMaxStages], ab_empty[kMaxStages], raw_full[kMaxRaw], raw_empty[kMaxRaw], done_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ float2 lut2[256];
    __shared__ int abort_flag;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool quantized = KIND != MAT_FP16;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t b_bytes = p.n_tile * BK * 2;
    const uint32_t stage_bytes = A_STAGE_BYTES + b_bytes;                   // [A | B], both 1024-byte aligned
    constexpr uint32_t raw_row = KIND == MAT_INT8 ? 64u : 32u;              // raw bytes per row and step
    const uint32_t raw_bytes = BM * raw_row;
    uint8_t* raw_base = smem + (size_t)p.stages * stage_bytes;              // raw weight stages
    uint8_t* scale_base = raw_base + (size_t)p.raw * raw_bytes;             // [2 groups][2 slots][BM][8 bytes]
    const uint32_t m0 = (blockIdx.x - grp.tile_start[gi]) * BM, n0 = blockIdx.y * p.n_tile;
    // this CTA's share of the K steps (split-K: grid.z CTAs per output tile)
    const uint32_t nk_all = p.K / BK;
    const uint32_t k_begin = (uint32_t)((uint64_t)nk_all * blockIdx.z / p.splits);
    const uint32_t nk = (uint32_t)((uint64_t)nk_all * (blockIdx.z + 1) / p.splits) - k_begin;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(&ab_full[s], quantized ? kDequantWarps / 2 + 1 : 2);  // one dequant group (or the weight TMA) + activation TMA
            mbar_init(&ab_empty[s], 1);
        }
        for (uint32_t r = 0; r < p.raw; ++r) {
            mbar_init(&raw_full[r], 1);
            mbar_init(&raw_empty[r], kDequantWarps / 2);
        }
        mbar_init(&done_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (KIND == MAT_NF4 && threadIdx.x < 256) lut2[threadIdx.x] = make_float2(p.table[threadIdx.x & 15], p.table[threadIdx.x >> 4]);
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(&tmem_base_slot)), "r"(p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = tmem_base_slot;

    if (warp < kDequantWarps) {
        if (quantized) {
            // ---- dequantizers: two groups of four warps take alternate pairs of steps (group g: steps 4j + 2g and
            // 4j + 2g + 1), so one group computes while the other sits in its fence and barriers; a thread owns a
            // row: 64 weights per step, one proxy fence and one round of arrivals per pair ----
            const uint32_t group = warp >> 2, row = threadIdx.x & (BM - 1);
            const uint32_t m = m0 + row;
            // scale slots cover 256 columns = four steps; the walk starts at a multiple of four steps
            const uint32_t nsuper = (nk + 3) / 4;
            const uint8_t* srow = reinterpret_cast<const uint8_t*>(p.scale) + ((size_t)m * (p.K / 256) + k_begin / 4) * 8;
            uint8_t* my_scale = scale_base + group * 2 * SCALE_SLOT_BYTES + row * 8;  // [group][2 slots][BM][8 bytes]
            cp_async8z(my_scale, srow, m < p.M);
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            for (uint32_t j = 0; j < nsuper; ++j) {
                if (j + 1 < nsuper) cp_async8z(my_scale + ((j + 1) & 1) * SCALE_SLOT_BYTES, srow + (size_t)(j + 1) * 8, m < p.M);
                asm volatile("cp.async.commit_group;\n" ::: "memory");
                asm volatile("cp.async.wait_group 1;\n" ::: "memory");
                const uint8_t* ss = my_scale + (j & 1) * SCALE_SLOT_BYTES;
                const uint32_t kt0 = 4 * j + 2 * group;
#pragma unroll 1
                for (uint32_t d = 0; d < 2; ++d) {
                    const uint32_t kt = kt0 + d;
                    if (kt >= nk) break;
                    const uint32_t r = kt % p.raw;
                    mbar_wait(&raw_full[r], (kt / p.raw) & 1, &abort_flag, p.status);
                    const uint4* rs = reinterpret_cast<const uint4*>(raw_base + (size_t)r * raw_bytes + row * raw_row);
                    const uint32_t s = kt % p.stages, use = kt / p.stages;
                    if (use > 0) mbar_wait(&ab_empty[s], (use - 1) & 1, &abort_flag, p.status);
                    uint8_t* sa = smem + (size_t)s * stage_bytes;
                    uint4 wv[4];
#pragma unroll
                    for (uint32_t h = 0; h < 2; ++h) {  // columns 32 h .. 32 h + 31 of the step
                        if (KIND == MAT_INT8)  // a 128-column block is two steps: this group's pair shares (min, max)
                            dequant_int8(rs[2 * h], rs[2 * h + 1], *reinterpret_cast<const uint32_t*>(ss + group * 4), wv);
                        else
                            dequant_nf4(rs[h], __half2float(*reinterpret_cast<const __half*>(ss + (kt & 3) * 2)), lut2, wv);
#pragma unroll
                        for (uint32_t c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(sa + sw128_offset(row, h * 4 + c)) = wv[c];
                    }
                    __syncwarp();  // every lane has consumed its raw bytes
                    if (lane == 0) mbar_arrive(&raw_empty[r]);  // the raw stage may be refilled
                }
                fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) {
                    if (kt0 < nk) mbar_arrive(&ab_full[kt0 % p.stages]);
                    if (kt0 + 1 < nk) mbar_arrive(&ab_full[(kt0 + 1) % p.stages]);
                }
            }
        }
        // ---- epilogue: TMEM -> registers -> activation -> token-major rows ----
        mbar_wait(&done_bar, 0, &abort_flag, p.status);
        tc_fence_after();
        const uint32_t quad = warp & 3, side = warp >> 2;  // lanes 32 quad .., half of the columns each
        const uint32_t m = m0 + quad * 32 + lane;
        const uint32_t c_begin = side * (p.n_tile / 2), c_end = c_begin + p.n_tile / 2;
        // split K: the partial tile goes to this CTA's own shared memory (the operand stages are free once every
        // MMA has completed), column-major [n_tile][BM] floats, for the cluster-wide sum below
        float* ws_mine = reinterpret_cast<float*>(smem);
        const size_t col_stride = p.out.stride[0], out_row = p.out.index(m < p.M ? m : 0, n0, 0);
        const bool act_none = p.act == WRK_ACT_NONE;
        // one CTA per output tile: the tile goes through shared memory when 16-byte pieces of a column are aligned in
        // the output (its first element of the tile 16-byte aligned, columns a multiple of 16 bytes apart)
        const uint32_t osize = p.out.dtype == WRK_F16 ? 2u : 4u;
        const bool staged = p.splits == 1 && (reinterpret_cast<uintptr_t>(p.out.base) + p.out.index(m0, n0, 0) * osize) % 16 == 0 &&
                            (col_stride * osize) % 16 == 0;
        // up to four 8-column accumulator loads are in flight before the single wait
        for (uint32_t c0 = c_begin; c0 < c_end; c0 += 32) {
            uint32_t v[4][8];
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q)
                if (c0 + 8 * q < c_end) tmem_ld8(tmem_d + ((quad * 32) << 16) + c0 + 8 * q, v[q]);
            tmem_ld_wait();
            if (!act_none && p.splits == 1) {  // the activation once, outside the store loops (which then hold no branch)
#pragma unroll
                for (uint32_t q = 0; q < 4; ++q)
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[q][j] = __float_as_uint(activate_f(p.act, __uint_as_float(v[q][j])));
            }
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q) {
                const uint32_t c = c0 + 8 * q;
                if (c >= c_end) continue;
                if (p.splits > 1) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) ws_mine[(size_t)(c + j) * BM + quad * 32 + lane] = __uint_as_float(v[q][j]);
                } else if (staged) {
                    // the finished values, in the output's type, into a [column][row] tile in shared memory
                    if (p.out.dtype == WRK_F16) {
                        __half* t = reinterpret_cast<__half*>(smem);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            t[(size_t)(c + j) * BM + quad * 32 + lane] =
                                __float2half_rn(__uint_as_float(v[q][j]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            ws_mine[(size_t)(c + j) * BM + quad * 32 + lane] =
                                __uint_as_float(v[q][j]);
                    }
                } else if (m < p.M) {
                    // element (m, n) of the output lies col_stride elements after (m, n - 1): one address, then steps
                    const size_t at = out_row + (size_t)c * col_stride;
                    if (p.out.dtype == WRK_F16) {
                        __half* o = static_cast<__half*>(p.out.base) + at;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (n0 + c + j < p.N) o[(size_t)j * col_stride] = __float2half_rn(__uint_as_float(v[q][j]));
                    } else {
                        float* o = static_cast<float*>(p.out.base) + at;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (n0 + c + j < p.N) o[(size_t)j * col_stride] = __uint_as_float(v[q][j]);
                    }
                }
            }
        }
        if (staged) {
            // ... and from there to global memory in 16-byte pieces: the 128 rows of a column are adjacent elements of
            // the output, so a warp writes whole 256- or 512-byte runs instead of 64 bytes per instruction
            asm volatile("bar.sync 1, %0;\n" ::"n"(kDequantWarps * 32) : "memory");
            const uint32_t esize = p.out.dtype == WRK_F16 ? 2u : 4u, per_col = BM * esize / 16, per_vec = 16 / esize;
            const uint32_t cols = min(p.n_tile, p.N - n0);
            const size_t col0 = p.out.index(m0, n0, 0);
            for (uint32_t i = threadIdx.x; i < cols * per_col; i += kDequantWarps * 32) {
                const uint32_t c = i / per_col, r = (i % per_col) * per_vec;  // column, first row of the piece
                if (m0 + r >= p.M) continue;
                const uint4 piece = *reinterpret_cast<const uint4*>(smem + ((size_t)c * BM + r) * esize);
                uint8_t* dst = static_cast<uint8_t*>(p.out.base) + (col0 + (size_t)c * col_stride + r) * esize;
                if (m0 + r + per_vec <= p.M) {
                    *reinterpret_cast<uint4*>(dst) = piece;
                } else {  // the matrix ends inside the piece
                    const uint8_t* src = reinterpret_cast<const uint8_t*>(&piece);
                    for (uint32_t e = 0; e < (p.M - m0 - r) * esize; ++e) dst[e] = src[e];
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---- MMA issuer ----
        const uint32_t idesc = f16_idesc(BM, p.n_tile);
        for (uint32_t kt = 0; kt < nk; ++kt) {
            const uint32_t s = kt % p.stages, use = kt / p.stages;
            mbar_wait(&ab_full[s], use & 1, &abort_flag, p.status);
            tc_fence_after();
            if (lane == 0) {
                const uint32_t sa = smem_addr(smem + (size_t)s * stage_bytes);
                const uint64_t da = sw128_desc(sa), db = sw128_desc(sa + A_STAGE_BYTES);
#pragma unroll
                for (uint32_t kk = 0; kk < BK / 16; ++kk)  // 32 bytes of K per instruction: + 2 in the address field
                    umma_f16(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (kt | kk) != 0 ? 1u : 0u);
                umma_commit(&ab_empty[s]);  // arrives when the MMAs above have read the stage
            }
            __syncwarp();
        }
        if (lane == 0) umma_commit(&done_bar);
        __syncwarp();
    } else if (warp == kWeightTmaWarp) {
        if (lane == 0) {
            if (quantized) {
                for (uint32_t kt = 0; kt < nk; ++kt) {
                    const uint32_t r = kt % p.raw, ruse = kt / p.raw;
                    if (ruse > 0) mbar_wait(&raw_empty[r], (ruse - 1) & 1, &abort_flag, p.status);
                    mbar_expect_tx(&raw_full[r], raw_bytes);
                    tma_load_2d(raw_base + (size_t)r * raw_bytes, &map_w, (k_begin + kt) * raw_row, m0, &raw_full[r]);
                }
            } else {
                for (uint32_t kt = 0; kt < nk; ++kt) {
                    const uint32_t s = kt % p.stages, use = kt / p.stages;
                    if (use > 0) mbar_wait(&ab_empty[s], (use - 1) & 1, &abort_flag, p.status);
                    mbar_expect_tx(&ab_full[s], A_STAGE_BYTES);
                    tma_load_2d(smem + (size_t)s * stage_bytes, &map_w, (k_begin + kt) * BK, m0, &ab_full[s]);
                }
            }
        }
    } else {
        if (lane == 0) {
            for (uint32_t kt = 0; kt < nk; ++kt) {
                const uint32_t s = kt % p.stages, use = kt / p.stages;
                if (use > 0) mbar_wait(&ab_empty[s], (use - 1) & 1, &abort_flag, p.status);
                mbar_expect_tx(&ab_full[s], b_bytes);
                tma_load_2d(smem + (size_t)s * stage_bytes + A_STAGE_BYTES, &map_x, (k_begin + kt) * BK, n0, &ab_full[s]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_d), "r"(p.tmem_cols) : "memory");
    }
    if (p.splits > 1) {
        // The CTAs of a cluster hold the partial tiles of one output tile.  After the cluster barrier CTA r adds
        // its share of the columns over all peers (in rank order: the sum does not depend on timing), through
        // distributed shared memory, and finishes those outputs.  The second barrier keeps every CTA's shared
        // memory alive until its peers have read it.  Both are hardware barriers that every thread reaches, also
        // after a wait above has given up.
        cluster_sync();
        const uint32_t rank = cluster_rank();
        {
            constexpr uint32_t kGroups = 4, kReduceThreads = kUmmaThreads;
            const uint32_t c_lo = p.n_tile * rank / p.splits, c_hi = p.n_tile * (rank + 1) / p.splits;
            const uint32_t v_lo = c_lo * (BM / 4), v_hi = c_hi * (BM / 4);  // groups of four rows
            const uint32_t base_addr = smem_addr(smem);
            const bool out_vec = reinterpret_cast<uintptr_t>(p.out.base) % 16 == 0;
            for (uint32_t base = v_lo; base < v_hi; base += kGroups * kReduceThreads) {
                float4 sum[kGroups];
#pragma unroll
                for (uint32_t u = 0; u < kGroups; ++u) sum[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (uint32_t z0 = 0; z0 < p.splits; z0 += 4) {
                    float4 v[kGroups][4];
#pragma unroll
                    for (uint32_t u = 0; u < kGroups; ++u) {
                        const uint32_t pos = base + u * kReduceThreads + threadIdx.x;
#pragma unroll
                        for (uint32_t dz = 0; dz < 4; ++dz) {
                            v[u][dz] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (pos < v_hi && z0 + dz < p.splits) v[u][dz] = ld_peer_smem(base_addr + pos * 16, z0 + dz);
                        }
                    }
#pragma unroll
                    for (uint32_t u = 0; u < kGroups; ++u)
#pragma unroll
                        for (uint32_t dz = 0; dz < 4; ++dz)
                            sum[u].x += v[u][dz].x, sum[u].y += v[u][dz].y, sum[u].z += v[u][dz].z, sum[u].w += v[u][dz].w;
                }
#pragma unroll
                for (uint32_t u = 0; u < kGroups; ++u) {
                    const uint32_t pos = base + u * kReduceThreads + threadIdx.x;
                    if (pos >= v_hi) continue;
                    const uint32_t c = pos / (BM / 4), row = (pos % (BM / 4)) * 4;
                    const uint32_t n = n0 + c, m = m0 + row;
                    if (n >= p.N) continue;
                    float r4[4] = {sum[u].x, sum[u].y, sum[u].z, sum[u].w};
                    if (p.act != WRK_ACT_NONE) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) r4[e] = activate_f(p.act, r4[e]);
                    }
                    const size_t at = p.out.index(m, n, 0);  // rows m .. m + 3 of a column are adjacent elements
                    if (m + 3 < p.M && (at & 3) == 0 && out_vec) {
                        if (p.out.dtype == WRK_F16) {
                            const __half2 lo = __floats2half2_rn(r4[0], r4[1]), hi = __floats2half2_rn(r4[2], r4[3]);
                            *reinterpret_cast<uint2*>(static_cast<__half*>(p.out.base) + at) = make_uint2(pack_half2(lo), pack_half2(hi));
                        } else {
                            *reinterpret_cast<float4*>(static_cast<float*>(p.out.base) + at) = make_float4(r4[0], r4[1], r4[2], r4[3]);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (m + e < p.M) dstore(p.out.base, p.out.dtype, at + e, r4[e]);
                    }
                }
            }
        }
        cluster_sync();
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry-point lookup: the library does not link libcuda.
EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

bool make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t rows, uint64_t row_bytes,
                 uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return false;
    const cuuint64_t gdim[2] = {inner, rows};
    const cuuint64_t gstride[1] = {row_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool matmul_umma_supported(const MatmulArgs& a) {
    if (a.B != 1 || a.N < 16 || a.M == 0) return false;
    if (a.K % BK != 0 || (a.kind != MAT_FP16 && a.K % 256 != 0)) return false;  // scale slots are fetched 8 bytes at a time
    if (reinterpret_cast<uintptr_t>(a.matrix) % 16 != 0) return false;
    if (a.scale != nullptr && reinterpret_cast<uintptr_t>(a.scale) % 8 != 0) return false;
    // activations go through a tensor map: fp16, rows 16-byte aligned
    if (a.in.dtype != WRK_F16 || a.in.stride[0] % 8 != 0) return false;
    const uintptr_t x0 = reinterpret_cast<uintptr_t>(a.in.base) + a.in.index(0, 0, 0) * 2;
    if (x0 % 16 != 0) return false;
    return encode_tiled() != nullptr;
}

bool matmul_umma_group_supported(const MatmulArgs* a, int count) {
    if (count < 1 || count > kMaxGroup) return false;
    for (int i = 0; i < count; ++i) {
        if (!matmul_umma_supported(a[i])) return false;
        if (a[i].kind != a[0].kind || a[i].K != a[0].K || a[i].N != a[0].N) return false;
    }
    return true;
}

cudaError_t matmul_umma_group(const MatmulArgs* args, int count, int32_t* status, cudaStream_t stream) {
    if (!matmul_umma_group_supported(args, count)) return cudaErrorInvalidValue;
    const MatmulArgs& a = args[0];
    UmmaGroup g{};
    g.count = (uint32_t)count;
    uint32_t row_tiles = 0;
    for (int i = 0; i < count; ++i) {
        g.tile_start[i] = row_tiles;
        row_tiles += (args[i].M + BM - 1) / BM;
    }
    for (int i = count; i <= kMaxGroup; ++i) g.tile_start[i] = row_tiles;
    UmmaParams p{};
    p.kind = a.kind;
    p.K = a.K;
    p.N = a.N;
    p.status = status;
    const uint32_t nk = a.K / BK;
    // Output tiles are 128 rows x n_tile tokens; K is split across the CTAs of a thread-block cluster while the
    // tiles alone leave SMs idle: a split keeps at least eight steps (a multiple of four, so scale slots stay
    // aligned), a cluster at most 8 CTAs.  Up to 512 tokens, 128-token tiles replace 256-token ones when that
    // doubles the CTAs of the single wave without lengthening a CTA's K walk: smaller operand stages (a deeper
    // ring) and smaller partial tiles.  (Measured: 2048x2048 Int8, 256 tokens: 22.8 -> 15.9 us; where the K walk
    // would double instead, 31 -> 37 us, so those keep 256.)
    int sms = 148, device = 0;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    auto splits_for = [&](uint32_t n_tile) {
        const uint32_t tiles = row_tiles * ((a.N + n_tile - 1) / n_tile);
        uint32_t want = std::max<uint32_t>(1, (uint32_t)sms / tiles);
        want = std::min<uint32_t>(want, std::max<uint32_t>(1, nk / 8));
        want = std::min<uint32_t>(want, 8);
        while (want > 1 && nk % (4 * want) != 0) --want;
        return want;
    };
    p.n_tile = std::min<uint32_t>(256, (a.N + 15) / 16 * 16);
    p.splits = splits_for(p.n_tile);
    if (p.n_tile > 128 && a.N <= 512) {
        const uint32_t s2 = splits_for(128);
        if (s2 >= p.splits && row_tiles * ((a.N + 127) / 128) * s2 <= (uint32_t)sms) p.n_tile = 128, p.splits = s2;
    }
    p.tmem_cols = 32;
    while (p.tmem_cols < p.n_tile) p.tmem_cols *= 2;
    const uint32_t stage_bytes = A_STAGE_BYTES + p.n_tile * BK * 2;
    const uint32_t raw_bytes = a.kind == MAT_INT8 ? BM * 64 : a.kind == MAT_NF4 ? BM * 32 : 0;
    // all of an SM's shared memory but the static part and the alignment slack: at 256-token tiles (48 KB operand
    // stages) that is four stages, one pair for each group of dequantizing warps, instead of three
    const uint32_t budget = 222u * 1024;
    p.raw = a.kind == MAT_FP16 ? 0 : std::min<uint32_t>(kMaxRaw, std::max<uint32_t>(2, nk));
    p.stages = std::min<uint32_t>(kMaxStages, std::max<uint32_t>(2, nk));
    while (p.stages * stage_bytes + p.raw * raw_bytes + 4 * SCALE_SLOT_BYTES > budget) {
        if (p.raw > 4) --p.raw;
        else if (p.stages > 4) --p.stages;
        else if (p.raw > 2) --p.raw;
        else if (p.stages > 2) --p.stages;
        else break;
    }
    if (p.splits > 1) {
        const uint32_t nk_split = nk / p.splits;
        p.stages = std::min<uint32_t>(p.stages, std::max<uint32_t>(2, nk_split));
        if (p.raw) p.raw = std::min<uint32_t>(p.raw, std::max<uint32_t>(2, nk_split));
    }

    for (int i = 0; i < count; ++i) {
        const MatmulArgs& ai = args[i];
        UmmaParams& pi = g.p[i];
        pi = p;
        pi.w = static_cast<const uint8_t*>(ai.matrix);
        pi.scale = ai.scale;
        pi.table = ai.table;
        pi.M = ai.M;
        pi.out = ai.out;
        pi.act = ai.act;
        bool ok;
        if (a.kind == MAT_FP16)
            ok = make_map_2d(&g.map_w[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, ai.matrix, a.K, ai.M, (uint64_t)a.K * 2, BK, BM,
                             CU_TENSOR_MAP_SWIZZLE_128B);
        else if (a.kind == MAT_INT8)
            ok = make_map_2d(&g.map_w[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, ai.matrix, a.K, ai.M, a.K, 64, BM, CU_TENSOR_MAP_SWIZZLE_NONE);
        else
            ok = make_map_2d(&g.map_w[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, ai.matrix, a.K / 2, ai.M, a.K / 2, 32, BM,
                             CU_TENSOR_MAP_SWIZZLE_NONE);
        const __half* x0 = static_cast<const __half*>(ai.in.base) + ai.in.index(0, 0, 0);
        ok = ok && make_map_2d(&g.map_x[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x0, a.K, a.N, (uint64_t)ai.in.stride[0] * 2, BK, p.n_tile,
                               CU_TENSOR_MAP_SWIZZLE_128B);
        if (!ok) return cudaErrorInvalidValue;
    }

    static SmemOptIn opt_in[3];
    auto kernel = a.kind == MAT_INT8 ? matmul_umma_kernel<MAT_INT8> : a.kind == MAT_NF4 ? matmul_umma_kernel<MAT_NF4> : matmul_umma_kernel<MAT_FP16>;
    if (cudaError_t e = opt_in[a.kind == MAT_INT8 ? 0 : a.kind == MAT_NF4 ? 1 : 2].ensure(kernel, 223 * 1024); e != cudaSuccess) return e;
    dim3 grid(row_tiles, (a.N + p.n_tile - 1) / p.n_tile, p.splits);
    size_t smem = (size_t)p.stages * stage_bytes + (size_t)p.raw * raw_bytes + 4 * SCALE_SLOT_BYTES + 1024;
    smem = std::max<size_t>(smem, (size_t)p.n_tile * BM * sizeof(float) + 1024);  // the partial tile / the staged output tile
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kUmmaThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = p.splits;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, g);
}

cudaError_t matmul_umma(const MatmulArgs& a, int32_t* status, cudaStream_t stream) { return matmul_umma_group(&a, 1, status, stream); }

}  // namespace k
}  // namespace wrk
