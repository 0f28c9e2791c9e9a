// The persistent decode kernel with its matrices on the 5th-generation tensor cores (TMA + tcgen05 + TMEM).
//
// The mma.sync weight loop of decode.cu spends about 250 warp instructions on every 2 KB of Int8 weights
// (copy issue, byte -> fp16 expansion, fragment loads, block-scale arithmetic): at 16 warps per SM it is bound
// by instruction issue at roughly half the HBM rate.  Here no thread touches a weight:
//   * four loader warps copy [rows][128 byte] blocks of the CTA's row range into a ring of 16 KB stages with
//     cp.async, 16 bytes per copy, straight into the 128-byte-swizzled operand layout; they take no part in the
//     phases and run ahead of the math across phase boundaries, because weights depend on nothing the job
//     computes.  (TMA boxes of this shape - 128 bytes is the widest a swizzled box can be - arrive at one
//     128-byte row per ~6 cycles per SM, measured the same from L2 as from HBM: 6.2 TB/s over the chip at best,
//     and 0.45 us per stage in this kernel.)
//   * four threads (one per SM sub-partition; a tcgen05.mma occupies its issuing thread for ~115 ns whatever its
//     N, and four issuers overlap) issue tcgen05.mma straight from shared memory: kind::i8 for Int8 matrices (the u8
//     weights as they are stored, against the activations as three signed base-256 digits per value, exact to
//     2^-23 of the largest activation of each 128-block), kind::f16 for fp16 matrices.  M = 128 stage rows
//     x N = 16 columns whose second group of eight aliases the first (stride 0): eight activation columns;
//   * the Int8 block scales enter after the MMA: every 128-weight block leaves a tile of s32 sums in tensor
//     memory; 128 threads (one per stage row) read their sums with tcgen05.ld and add
//     (max - min) / 255 * step * sum + min * (sum of the block's activations) in f32.
// Row ranges shorter than 128 rows pack several k-blocks into one stage (4 blocks of <= 32 rows, 2 of <= 64):
// stage row L holds row L % P of block L / P, each block is multiplied against its own activation columns into
// its own accumulator, and lane L keeps the sum of its row over its blocks; the partial sums of a row meet in
// shared memory at the end.
// The loader warps (16..19) never join the compute warps' barriers: those are barrier 0 over 512 threads.
#define WRK_CTA_SYNC() asm volatile("bar.sync 0, 512;\n" ::: "memory")
#include "decode_step_common.cuh"

#include <cstdlib>
#include <cstring>

namespace wrk {
namespace k {

namespace {

constexpr int kMaxSlots = 12;               // a multiple of kIssuers
constexpr uint32_t kSlotBytes = 16384;      // 128 rows x 128 bytes
constexpr int kIssuers = 4;                 // lane 0 of warps 4..7: stage g is multiplied by issuer g % 4
constexpr int kIssuerWarp0 = 4;
constexpr int kDrainGroups = 3;  // warps 0-3, 8-11, 12-15 read Int8 accumulators
constexpr int kLoaderWarp0 = 16;            // the warps after the compute warps
constexpr int kLoaders = 128;               // loader threads
constexpr int kUmmaThreads = kThreads + kLoaders;
constexpr uint32_t kTmemCols = 256;         // Int8: 4 issuers x 2 x 16 columns; fp16: 2 tiles x 4 issuers x 16 columns
constexpr uint32_t kF16Cols = 128;          // first column of the fp16 accumulators
constexpr float kDigitScale = 8323072.0f;   // 127 * 65536: |value / step| fits three balanced base-256 digits

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// K-major, 128-byte swizzle: rows of 128 bytes, groups of 8 rows `sbo` bytes apart (0: every group is the first).
__device__ __forceinline__ uint64_t sw128_desc(uint32_t saddr, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
template <bool I8>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if (I8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t v[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void bar_sync_128() { asm volatile("bar.sync 2, 128;\n" ::: "memory"); }
__device__ __forceinline__ void bar_sync_drain() { asm volatile("bar.sync 4, %0;\n" ::"n"(kDrainGroups * 128) : "memory"); }

// The CTA's pipeline state, in shared memory.  Stages are numbered from the start of the kernel: stage g sits in
// slot g % num_slots, is multiplied by issuer g % 4 and (Int8) leaves its sums in that issuer's buffer (g / 4) % 2.
struct Pipe {
    uint64_t slot_full[kMaxSlots], slot_empty[kMaxSlots];
    uint64_t i8_full[kIssuers][2], i8_empty[kIssuers][2];  // one commit / four warp arrivals
    uint64_t f16_full[2], f16_empty[2];                    // four commits (one per issuer) / four warp arrivals
    uint32_t issued;            // stages requested since the kernel began (loader thread 0)
    uint32_t loaders_done;      // loader threads that have left, with none of their copies in flight
    uint32_t stage_base;        // first stage of the phase in progress (every role reads it after a barrier)
    uint32_t i8_base;           // Int8 stages before the phase in progress: stage n of them is multiplied by issuer
                                // n % 4 into its buffer (n / 4) % 2
    uint32_t stage_end;         // one past the last stage whose MMAs have been issued or are being issued
    uint32_t f16_tiles;         // fp16 tiles handed over since the kernel began
    uint32_t tmem;
    int32_t abort_flag;
};

using Tile = UmmaTile;
__device__ __forceinline__ Tile tile_of(const UmmaWork& wk, int tile, uint32_t T) {
    return umma_tile(wk.r1 - wk.r0, tile, wk.kind, wk.K, T);
}
__device__ __forceinline__ int stages_of(const UmmaWork& wk, uint32_t T) {
    const int total = wk.r1 - wk.r0;
    if (total <= 0) return 0;
    const int ntiles = (total + 127) / 128;
    int n = (ntiles - 1) * tile_of(wk, 0, T).nslots;
    return n + tile_of(wk, ntiles - 1, T).nslots;
}

// A bounded wait on an mbarrier phase by one thread.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, Pipe* pipe, int32_t* status) {
    for (uint32_t i = 0; i < kStepSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*reinterpret_cast<volatile int32_t*>(&pipe->abort_flag)) return false;
    }
    pipe->abort_flag = 1;
    atomicExch(status, (int32_t)WRK_ERR_TIMEOUT);
    return false;
}

// The same wait by a whole warp: lane 0 watches the barrier, the others wait for its answer.
__device__ __forceinline__ bool wait_bar_warp(uint64_t* bar, uint32_t parity, Pipe* pipe, int32_t* status) {
    bool ok = true;
    if ((threadIdx.x & 31u) == 0 && !mbar_try_wait(bar, parity)) {
        ok = false;
        for (uint32_t i = 0; i < kStepSpinLimit; ++i) {
            if (mbar_try_wait(bar, parity)) {
                ok = true;
                break;
            }
            if (*reinterpret_cast<volatile int32_t*>(&pipe->abort_flag)) break;
            if (i + 1 == kStepSpinLimit) {
                pipe->abort_flag = 1;
                atomicExch(status, (int32_t)WRK_ERR_TIMEOUT);
            }
        }
    }
    return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
}

// The loaders: 128 threads copy every stage of the job in order, each as soon as its slot is free.  A thread
// attaches its copies of a stage to the slot's `slot_full` barrier (cp.async.mbarrier.arrive.noinc: one arrival
// per loader thread, made by the hardware when the thread's copies have landed), so no loader ever waits for data.
// The issuer that takes the stage fences the generic-proxy writes against the tensor cores' async-proxy reads.
// A wait for a slot ends when the MMAs that read the slot's previous stage complete, which can lie several phases
// ahead: it is bounded by time (about two seconds) and ends at once when another wait of the CTA has given up.
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __noinline__ void load_stages(Pipe* pipe, const UmmaWork* work, int num_gemv, int num_slots, uint32_t T, uint8_t* slots,
                                         int32_t* status, uint32_t lt) {
    uint32_t g = 0, ring = 0, wrapped = 0;
    bool alive = true;
    for (int entry = 0; alive && entry < num_gemv; ++entry) {
        const UmmaWork wk = work[entry];
        const int total = wk.r1 - wk.r0;
        if (total <= 0 || wk.direct) continue;
        const int ntiles = (total + 127) / 128;
        const size_t pitch = wk.kind == MAT_INT8 ? (size_t)wk.K : (size_t)wk.K * 2;
        for (int tile = 0; alive && tile < ntiles; ++tile) {
            const Tile t = tile_of(wk, tile, T);
            // This thread copies the 16-byte column lt % 8 of eight stage rows: with R = P / 16 row steps per
            // k-block, copy u is row lt / 8 + 16 (u % R) of block u / R.  Source offsets and (swizzled) stage
            // offsets are the same for every stage of the tile.
            const uint32_t col = lt & 7u, r_first = lt >> 3;
            const uint32_t R = (uint32_t)t.P / 16u;
            const uint8_t* src0 = wk.w + (size_t)(wk.r0 + tile * 128) * pitch + col * 16;
            uint32_t soff[8], doff[8];
            uint32_t live = 0;  // bit u: the row exists; bits 8 + u / R ...: compared with the stage's block count below
#pragma unroll
            for (uint32_t u = 0; u < 8; ++u) {
                const uint32_t i = u / R, r = r_first + 16u * (u % R);
                const uint32_t srow = i * (uint32_t)t.P + r;  // stage row: 8-row atoms of 1 KB, chunk ^ row % 8
                soff[u] = i * 128u + r * (uint32_t)pitch;
                doff[u] = (srow >> 3) * 1024u + (srow & 7u) * 128u + ((col ^ (srow & 7u)) << 4);
                if (r < (uint32_t)t.rows) live |= 1u << u;
            }
            for (int j = 0; alive && j < t.nslots; ++j) {
                if (wrapped != 0) {
                    // one lane per warp watches the barrier; the others wait for it
                    const uint32_t parity = (wrapped - 1u) & 1u;
                    bool ok = true;
                    if ((lt & 31u) == 0 && !mbar_try_wait(&pipe->slot_empty[ring], parity)) {
                        const unsigned long long t0 = global_timer();
                        for (;;) {
                                            if (mbar_try_wait(&pipe->slot_empty[ring], parity)) break;
                            if (*reinterpret_cast<volatile int32_t*>(&pipe->abort_flag)) {
                                ok = false;
                                break;
                            }
                            if (global_timer() - t0 > 2000000000ull) {
                                pipe->abort_flag = 1;
                                atomicExch(status, (int32_t)WRK_ERR_TIMEOUT);
                                ok = false;
                                break;
                            }
                        }
                    }
                    alive = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!alive) break;
                }
                const uint32_t q = (uint32_t)min(t.Q, t.nkb - j * t.Q);
                uint8_t* dst = slots + (size_t)ring * kSlotBytes;
                const uint8_t* src = src0 + (size_t)(j * t.Q) * 128;
#pragma unroll
                for (uint32_t u = 0; u < 8; ++u)
                    if (((live >> u) & 1u) != 0 && u / R < q) cp_async16z(dst + doff[u], src + soff[u], true);
                cp_async_arrive(&pipe->slot_full[ring]);
                ++g;
                if (lt == 0) *reinterpret_cast<volatile uint32_t*>(&pipe->issued) = g;
                if (++ring == (uint32_t)num_slots) {
                    ring = 0;
                    ++wrapped;
                }
            }
        }
    }
    // nothing of this thread in flight when it leaves
    asm volatile("cp.async.wait_all;\n" ::: "memory");
    atomicAdd(&pipe->loaders_done, 1u);
}

// Offset of (stage j, operand row n, 16-byte chunk) in the activation operand; `atom` bytes per stage: one 8-row
// atom when the stage's activation rows fit it (the MMA's second group of eight columns then aliases the first),
// else two.
__device__ __forceinline__ uint32_t operand_offset(uint32_t j, uint32_t n, uint32_t chunk, uint32_t atom) {
    return j * atom + (n >> 3) * 1024u + (n & 7u) * 128u + ((chunk ^ (n & 7u)) << 4);
}

// Activations of an Int8 matrix as three signed base-256 digits per value, step = (largest |x| of the 128-block)
// / (127 * 65536).  k-block kb = Q j + i is block i of stage j: digit d of token t is operand row i * 3 T + 3 t + d
// of the stage.  bconst[t][kb] = (step, sum of the block's activations).
__device__ __forceinline__ void digitize(const __half* x, uint32_t x_stride, uint32_t T, uint32_t K, int Q, uint32_t atom,
                                         uint8_t* breg, float2* bconst, uint32_t nkb_max) {
    const uint32_t groups = K / 8;
    const uint32_t lane16 = threadIdx.x & 15;
    const uint32_t half_warp = 0xffffu << (threadIdx.x & 16);  // the 16 lanes of one 128-block enter and leave the loop together
    for (uint32_t t = 0; t < T; ++t) {
        for (uint32_t gi = threadIdx.x; gi < groups; gi += kThreads) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)t * x_stride + gi * 8);
            const __half2* h = reinterpret_cast<const __half2*>(&raw);
            float v[8];
            float m = 0.f, sum = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]);
                v[2 * e] = f.x;
                v[2 * e + 1] = f.y;
                m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
                sum += f.x + f.y;
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) {
                m = fmaxf(m, __shfl_xor_sync(half_warp, m, off, 16));
                sum += __shfl_xor_sync(half_warp, sum, off, 16);
            }
            const bool finite = m > 0.f && m < 3.0e38f;
            const float inv = finite ? kDigitScale / m : 0.f;
            // X + 0x808080 adds 128 at every digit position, carries included: its bytes are the balanced digits + 128,
            // and the xor turns each into the digit as a signed byte
            uint32_t wv[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) wv[e] = (uint32_t)(__float2int_rn(v[e] * inv) + 0x808080) ^ 0x808080u;
            uint32_t d0[2], d1[2], d2[2];
#pragma unroll
            for (int hq = 0; hq < 2; ++hq) {
                const uint32_t a = wv[4 * hq], b = wv[4 * hq + 1], c = wv[4 * hq + 2], d = wv[4 * hq + 3];
                d0[hq] = __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
                d1[hq] = __byte_perm(__byte_perm(a, b, 0x0051), __byte_perm(c, d, 0x0051), 0x5410);
                d2[hq] = __byte_perm(__byte_perm(a, b, 0x0062), __byte_perm(c, d, 0x0062), 0x5410);
            }
            const uint32_t kb = gi >> 4;
            const uint32_t j = kb / (uint32_t)Q, i = kb % (uint32_t)Q;
            const uint32_t chunk = lane16 >> 1, half8 = (lane16 & 1) * 8;
            const uint32_t r = i * 3 * T + 3 * t;
            *reinterpret_cast<uint2*>(breg + operand_offset(j, r + 0, chunk, atom) + half8) = make_uint2(d0[0], d0[1]);
            *reinterpret_cast<uint2*>(breg + operand_offset(j, r + 1, chunk, atom) + half8) = make_uint2(d1[0], d1[1]);
            *reinterpret_cast<uint2*>(breg + operand_offset(j, r + 2, chunk, atom) + half8) = make_uint2(d2[0], d2[1]);
            if (lane16 == 0) bconst[t * nkb_max + kb] = make_float2(finite ? m / kDigitScale : 0.f, sum);
        }
    }
}

// Activations of an fp16 matrix: token t of k-block kb = Q j + i (64 values) is operand row i * T + t of stage j.
__device__ __forceinline__ void stage_fp16(const __half* x, uint32_t x_stride, uint32_t T, uint32_t K, int Q, uint32_t atom,
                                           uint8_t* breg) {
    const uint32_t groups = K / 8;
    for (uint32_t t = 0; t < T; ++t)
        for (uint32_t gi = threadIdx.x; gi < groups; gi += kThreads) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)t * x_stride + gi * 8);
            const uint32_t kb = gi >> 3, chunk = gi & 7;
            const uint32_t j = kb / (uint32_t)Q, i = kb % (uint32_t)Q;
            *reinterpret_cast<uint4*>(breg + operand_offset(j, i * T + t, chunk, atom)) = raw;
        }
}

// One issuer's side of a row range: multiply its stages (every fourth), hand the accumulators over.
template <bool I8>
__device__ __noinline__ void issue_mmas(Pipe* pipe, const UmmaWork wk, uint32_t T, int num_slots, uint8_t* slots, uint8_t* breg, int w,
                                        int32_t* status) {
    const uint32_t idesc = I8 ? ((2u << 4) | (1u << 10) | (2u << 17) | (8u << 24)) : ((1u << 4) | (2u << 17) | (8u << 24));
    const uint32_t tmem = pipe->tmem;
    const int ntiles = (wk.r1 - wk.r0 + 127) / 128;
    uint32_t g = pipe->stage_base;
    uint32_t n8 = pipe->i8_base;  // Int8: the stage's number among the Int8 stages
    uint32_t ft = pipe->f16_tiles;
    uint32_t ring = g % (uint32_t)num_slots, wrapped = g / (uint32_t)num_slots;  // slot of stage g, wraps before it
    for (int tile = 0; tile < ntiles; ++tile) {
        const Tile t = tile_of(wk, tile, T);
        const uint32_t sbo = t.atom == 1024u ? 0u : 1024u;
        const uint32_t tb = ft & 1u;
        bool first = true;
        if (!I8 && ft >= 2 && !wait_bar(&pipe->f16_empty[tb], ((ft >> 1) - 1u) & 1u, pipe, status)) return;
        for (int j = 0; j < t.nslots; ++j, ++g, ++n8) {
            const uint32_t n = I8 ? n8 : g;
            const uint32_t s = ring, full_parity = wrapped & 1u;
            if (++ring == (uint32_t)num_slots) {
                ring = 0;
                ++wrapped;
            }
            if ((int)(n & 3u) != w) continue;
            if (!wait_bar(&pipe->slot_full[s], full_parity, pipe, status)) return;
            const uint32_t u = (n >> 2) & 1u;
            if (I8 && n >= 8 && !wait_bar(&pipe->i8_empty[w][u], ((n >> 3) - 1u) & 1u, pipe, status)) return;
            fence_async_smem();  // the loaders' copies (generic proxy), observed through the barrier, before the MMAs' reads
            tc_fence_after();
            const uint64_t da = sw128_desc(smem_u32(slots + (size_t)s * kSlotBytes), 1024);
            const uint64_t db = sw128_desc(smem_u32(breg + (size_t)j * t.atom), sbo);
            const uint32_t d = I8 ? tmem + (uint32_t)(w * 2 + (int)u) * 16u : tmem + kF16Cols + tb * 64u + (uint32_t)w * 16u;
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk)  // 32 bytes of K per instruction: + 2 in the address field
                umma<I8>(d, da + 2 * kk, db + 2 * kk, idesc, I8 ? (kk != 0) : (!first || kk != 0));
            first = false;
            umma_commit(&pipe->slot_empty[s]);  // arrives when the MMAs above have read the stage
            if (I8) umma_commit(&pipe->i8_full[w][u]);
        }
        if (!I8) {
            umma_commit(&pipe->f16_full[tb]);  // one arrival per issuer, with or without stages of its own
            ++ft;
        }
    }
}

// The 128 accumulator lanes' side: warps 0-3, thread L owns stage row L = (k-block L / P of the stage, row L % P).
template <bool I8>
__device__ __noinline__ void drain_accumulators(Pipe* pipe, const GemvCore& a, const UmmaWork wk, const float2* bconst, uint32_t nkb_max,
                                                float* part, int32_t* status) {
    // Int8: kDrainGroups groups of four warps take the stages in turn (a stage's handshake with the tensor cores is a
    // chain of latencies, about half a microsecond; one group alone would pace the weight stream); fp16: group 0 only,
    // once per tile.  A warp reads the TMEM lanes 32 * (warp % 4) onwards, so every group sees all 128 rows.
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t grp = I8 ? (warp < 4 ? 0u : (warp - 4u) >> 2) : 0u;
    constexpr uint32_t ND = I8 ? (uint32_t)kDrainGroups : 1u;
    const uint32_t L = threadIdx.x & 127u;
    const GemvProblem& p = a.p[wk.problem];
    const uint32_t T = a.T;
    const int epi = a.epilogue;
    const uint32_t tmem = pipe->tmem + (((warp & 3u) * 32u) << 16);
    const int ntiles = (wk.r1 - wk.r0 + 127) / 128;
    uint32_t g = I8 ? pipe->i8_base : pipe->stage_base;
    uint32_t ft = pipe->f16_tiles;
    for (int tile = 0; tile < ntiles; ++tile) {
        const Tile t = tile_of(wk, tile, T);
        const uint32_t i = L / (uint32_t)t.P, lrow = L % (uint32_t)t.P;
        const bool row_ok = (int)lrow < t.rows;
        const uint32_t row = (uint32_t)(wk.r0 + tile * 128) + lrow;
        // the row's epilogue operands go in flight before the stages are drained
        const bool owner = grp == 0 && i == 0 && row_ok;
        EpiOperands eo[2];
        if (owner)
            for (uint32_t tok = 0; tok < T; ++tok) eo[tok] = epilogue_fetch_rt(epi, a, p, row, (int)tok);
        float acc[2] = {0.f, 0.f};
        if (I8) {
            const uint32_t* sp = reinterpret_cast<const uint32_t*>(wk.scale) + (size_t)(row_ok ? row : (uint32_t)wk.r0) * t.nkb;
            // this group's stages are grp, grp + ND, ...; their block scales four of them ahead
            uint32_t mm[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int kb = (int)(grp + (uint32_t)u * ND) * t.Q + (int)i;
                mm[u] = kb < t.nkb ? __ldg(sp + kb) : 0u;
            }
            for (int j0 = (int)grp; j0 < t.nslots; j0 += 4 * (int)ND) {
                uint32_t nx[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int kb = (j0 + (4 + u) * (int)ND) * t.Q + (int)i;
                    nx[u] = kb < t.nkb ? __ldg(sp + kb) : 0u;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = j0 + u * (int)ND;
                    if (j >= t.nslots) break;
                    const uint32_t gj = g + (uint32_t)j;
                    const uint32_t w = gj & 3u, ub = (gj >> 2) & 1u;
                    // a wait that gave up is skipped by the whole warp; the loop and its barriers still run to the end
                    const bool ok = wait_bar_warp(&pipe->i8_full[w][ub], (gj >> 3) & 1u, pipe, status);
                    uint32_t v[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) v[e] = 0;
                    if (ok) {
                        tc_fence_after();
                        tmem_ld16(tmem + (w * 2u + ub) * 16u, v);
                        tmem_ld_wait();
                        tc_fence_before();
                        __syncwarp();
                        if ((L & 31u) == 0) mbar_arrive(&pipe->i8_empty[w][ub]);
                    }
                    const int kb = j * t.Q + (int)i;
                    if (kb < t.nkb) {
                        const float2 mnmx = __half22float2(*reinterpret_cast<const __half2*>(&mm[u]));
                        const float sc = (mnmx.y - mnmx.x) * (1.0f / 255.0f);
#pragma unroll
                        for (uint32_t tok = 0; tok < 2; ++tok) {
                            if (tok >= T) break;
                            // this lane's block: columns [i * 3 T + 3 tok, + 3)
                            int d0 = 0, d1 = 0, d2 = 0;
#pragma unroll
                            for (uint32_t ii = 0; ii < 4; ++ii) {
                                const uint32_t c = ii * 3u * T + 3u * tok;
                                if (ii == i && c + 2u < 16u) {
                                    d0 = (int)v[c];
                                    d1 = (int)v[c + 1];
                                    d2 = (int)v[c + 2];
                                }
                            }
                            const float2 bc = bconst[tok * nkb_max + (uint32_t)kb];
                            const float V = fmaf((float)d2, 65536.0f, fmaf((float)d1, 256.0f, (float)d0));
                            acc[tok] = fmaf(sc * bc.x, V, fmaf(mnmx.x, bc.y, acc[tok]));
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) mm[u] = nx[u];
            }
            g += (uint32_t)t.nslots;
        } else {
            const uint32_t gtile = g;
            g += (uint32_t)t.nslots;
            const uint32_t tb = ft & 1u;
            const bool ok = wait_bar_warp(&pipe->f16_full[tb], (ft >> 1) & 1u, pipe, status);
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (uint32_t w = 0; w < (uint32_t)kIssuers; ++w) {
                    uint32_t v[16];
                    tmem_ld16(tmem + kF16Cols + tb * 64u + w * 16u, v);
                    tmem_ld_wait();
                    // issuer w multiplied the stages whose number is w modulo 4: it has sums of this tile if one of
                    // the tile's stages is among them (every stage of an fp16 tile holds all Q blocks)
                    if (((w - gtile) & 3u) < (uint32_t)t.nslots) {
#pragma unroll
                        for (uint32_t tok = 0; tok < 2; ++tok) {
                            if (tok >= T) break;
#pragma unroll
                            for (uint32_t ii = 0; ii < 4; ++ii)
                                if (ii == i && ii * T + tok < 16u) acc[tok] += __uint_as_float(v[ii * T + tok]);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if ((L & 31u) == 0) mbar_arrive(&pipe->f16_empty[tb]);
            }
            ++ft;
        }
        // a row's blocks and the groups' shares meet: lane L of group 0 adds the lanes L + P, L + 2 P, ... of every group
        float* mine = part + grp * 256u;
        mine[L] = row_ok ? acc[0] : 0.f;
        mine[128 + L] = row_ok ? acc[1] : 0.f;
        if (I8) bar_sync_drain();
        else bar_sync_128();
        if (owner) {
            for (uint32_t tok = 0; tok < T; ++tok) {
                float total = 0.f;
                for (uint32_t d = 0; d < ND; ++d)
                    for (int b = 0; b < t.Q; ++b) total += part[d * 256u + tok * 128u + L + (uint32_t)(b * t.P)];
                epilogue_one_rt(epi, a, p, row, (int)tok, total, eo[tok]);
            }
        }
        // `part` is written again by the next tile
        if (I8) bar_sync_drain();
        else bar_sync_128();
    }
}

// ---- one-token prologue in registers ---------------------------------------------------------------
// Layer norm (+ token shift) of the job's single token with every value in registers: thread t owns channels
// [8 t, 8 t + 8).  What does not depend on the previous phase (norm weight and bias, shift factors, the carry row
// of the token's sequence) is loaded before the grid barrier; after it come the row itself, two block sums (mean,
// then variance about the mean, as the reference's layer norm computes them) and the arithmetic.  The shifted
// vectors are rounded to fp16 like the tensors the reference stores them in.
constexpr int kFastMaxC = 8 * kThreads;
struct FastParams {
    uint4 w, b, mix[2];
    float prev[8];
};
__device__ __forceinline__ void fast_prologue_load(const GemvCore& a, int nv, FastParams& fp) {
    const uint32_t c0 = threadIdx.x * 8;
    if (c0 >= a.C) return;
    fp.w = *reinterpret_cast<const uint4*>(a.ln_w + c0);
    fp.b = *reinterpret_cast<const uint4*>(a.ln_b + c0);
    if (nv > 0) {
        fp.mix[0] = *reinterpret_cast<const uint4*>(a.mix0 + c0);
        if (nv > 1) fp.mix[1] = *reinterpret_cast<const uint4*>(a.mix1 + c0);
        const CursorD cu = cursor_at(a.cursors, a.wide, 0);
        const float* st = static_cast<const float*>(a.state.base) + a.state.index(c0, 0, cu.batch);
        const float4 p0 = *reinterpret_cast<const float4*>(st), p1 = *reinterpret_cast<const float4*>(st + 4);
        fp.prev[0] = p0.x; fp.prev[1] = p0.y; fp.prev[2] = p0.z; fp.prev[3] = p0.w;
        fp.prev[4] = p1.x; fp.prev[5] = p1.y; fp.prev[6] = p1.z; fp.prev[7] = p1.w;
    }
}
// out[v][e]: vector v (the normalised row when nv == 0, else the shifted vectors) of this thread's channels.
__device__ __forceinline__ void fast_prologue_run(const GemvCore& a, int nv, const FastParams& fp, float* scratch, float out[2][8]) {
    const uint32_t c0 = threadIdx.x * 8;
    const bool on = c0 < a.C;
    float v[8];
    float sum = 0.f;
    if (on) {
        const uint4 raw = *reinterpret_cast<const uint4*>(a.ln_x + (size_t)a.ln_row_off[0] * a.C + c0);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(h[e]);
            v[2 * e] = f.x;
            v[2 * e + 1] = f.y;
            sum += f.x + f.y;
        }
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = 0.f;
    }
    const float mean = block_sum_256(sum, scratch) / (float)a.C;
    float m2 = 0.f;
    if (on)
#pragma unroll
        for (int e = 0; e < 8; ++e) m2 += (v[e] - mean) * (v[e] - mean);
    const float dev = rsqrtf(block_sum_256(m2, scratch + kWarps) / (float)a.C + a.ln_eps);
    if (!on) return;
    const __half* wh = reinterpret_cast<const __half*>(&fp.w);
    const __half* bh = reinterpret_cast<const __half*>(&fp.b);
    uint4 normed;
    __half* nh = reinterpret_cast<__half*>(&normed);
#pragma unroll
    for (int e = 0; e < 8; ++e) nh[e] = __float2half_rn(fmaf((v[e] - mean) * dev, __half2float(wh[e]), __half2float(bh[e])));
    if (a.ln_out != nullptr && blockIdx.x == 0) *reinterpret_cast<uint4*>(a.ln_out + c0) = normed;
    if (nv == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) out[0][e] = __half2float(nh[e]);
        return;
    }
    for (int vi = 0; vi < nv; ++vi) {
        const __half* fh = reinterpret_cast<const __half*>(&fp.mix[vi]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float cur = __half2float(nh[e]), f = __half2float(fh[e]);
            const float lhs = a.reversed ? cur : fp.prev[e], rhs = a.reversed ? fp.prev[e] : cur;
            out[vi][e] = __half2float(__float2half_rn(lhs * (1.0f - f) + rhs * f));
        }
    }
}
// This thread's eight values (k = 8 t ...) as the activation operand: digits (Int8) or fp16.
__device__ __forceinline__ void fast_stage(const float x[8], bool active, bool i8, int Q, uint32_t atom, uint8_t* breg,
                                           float2* bconst) {
    const uint32_t gi = threadIdx.x;
    const uint32_t lane16 = threadIdx.x & 15;
    if (!i8) {
        if (!active) return;
        uint4 raw;
        __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(x[2 * e], x[2 * e + 1]);
        const uint32_t kb = gi >> 3, chunk = gi & 7;
        const uint32_t j = kb / (uint32_t)Q, i = kb % (uint32_t)Q;
        *reinterpret_cast<uint4*>(breg + operand_offset(j, i, chunk, atom)) = raw;
        return;
    }
    // whole half-warps are active or not (C is a multiple of 128)
    if (!active) return;
    const uint32_t half_warp = 0xffffu << (threadIdx.x & 16);
    float m = 0.f, sum = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        m = fmaxf(m, fabsf(x[e]));
        sum += x[e];
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) {
        m = fmaxf(m, __shfl_xor_sync(half_warp, m, off, 16));
        sum += __shfl_xor_sync(half_warp, sum, off, 16);
    }
    const bool finite = m > 0.f && m < 3.0e38f;
    const float inv = finite ? kDigitScale / m : 0.f;
    uint32_t wv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) wv[e] = (uint32_t)(__float2int_rn(x[e] * inv) + 0x808080) ^ 0x808080u;
    uint32_t d0[2], d1[2], d2[2];
#pragma unroll
    for (int hq = 0; hq < 2; ++hq) {
        const uint32_t aa = wv[4 * hq], bb = wv[4 * hq + 1], cc = wv[4 * hq + 2], dd = wv[4 * hq + 3];
        d0[hq] = __byte_perm(__byte_perm(aa, bb, 0x0040), __byte_perm(cc, dd, 0x0040), 0x5410);
        d1[hq] = __byte_perm(__byte_perm(aa, bb, 0x0051), __byte_perm(cc, dd, 0x0051), 0x5410);
        d2[hq] = __byte_perm(__byte_perm(aa, bb, 0x0062), __byte_perm(cc, dd, 0x0062), 0x5410);
    }
    const uint32_t kb = gi >> 4;
    const uint32_t j = kb / (uint32_t)Q, i = kb % (uint32_t)Q;
    const uint32_t chunk = lane16 >> 1, half8 = (lane16 & 1) * 8;
    const uint32_t r = i * 3;
    *reinterpret_cast<uint2*>(breg + operand_offset(j, r + 0, chunk, atom) + half8) = make_uint2(d0[0], d0[1]);
    *reinterpret_cast<uint2*>(breg + operand_offset(j, r + 1, chunk, atom) + half8) = make_uint2(d1[0], d1[1]);
    *reinterpret_cast<uint2*>(breg + operand_offset(j, r + 2, chunk, atom) + half8) = make_uint2(d2[0], d2[1]);
    if (lane16 == 0) bconst[kb] = make_float2(finite ? m / kDigitScale : 0.f, sum);
}

__global__ void __launch_bounds__(kUmmaThreads, 1) decode_step_umma_kernel(const UmmaStepArgs s) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ float scratch[2 * kWarps];
    __shared__ __align__(16) StepPhase desc[2];
    __shared__ __align__(8) uint64_t desc_bar[2];
    __shared__ __align__(8) Pipe pipe;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* slots = smem;
    uint8_t* breg = slots + (size_t)s.num_slots * kSlotBytes;            // activation operand (8 / 16-row atoms)
    __half* xs = reinterpret_cast<__half*>(breg + s.b_bytes - s.x_bytes);  // prologue rows, at the region's end
    float2* bconst = reinterpret_cast<float2*>(breg + s.b_bytes);        // [2][nkb_max]
    float* part = reinterpret_cast<float*>(bconst + 2 * s.nkb_max);      // [kDrainGroups][2][128]
    // this CTA's row ranges, one per multiply phase: read from global memory where they are needed (64 bytes each,
    // long before the data they describe)
    const UmmaWork* work = s.work + (size_t)blockIdx.x * s.num_gemv;
    GridSync gs{s.barrier, s.status, s.timeline, &abort_flag, 0};

    if (threadIdx.x == 0) {
        abort_flag = 0;
        pipe.abort_flag = 0;
        pipe.issued = pipe.loaders_done = pipe.stage_base = pipe.i8_base = pipe.stage_end = pipe.f16_tiles = 0;
        mbar_init(&desc_bar[0], 1);
        mbar_init(&desc_bar[1], 1);
        for (int i = 0; i < kMaxSlots; ++i) {
            mbar_init(&pipe.slot_full[i], kLoaders);
            mbar_init(&pipe.slot_empty[i], 1);
        }
        for (int w = 0; w < kIssuers; ++w)
            for (int u = 0; u < 2; ++u) {
                mbar_init(&pipe.i8_full[w][u], 1);
                mbar_init(&pipe.i8_empty[w][u], 4);  // one arrival per accumulator-lane warp
            }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&pipe.f16_full[i], kIssuers);
            mbar_init(&pipe.f16_empty[i], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        fence_async_smem();
        for (int i = 0; i < 2 && i < s.num_phases; ++i) {
            mbar_expect_tx(&desc_bar[i], (uint32_t)sizeof(StepPhase));
            bulk_load(&desc[i], s.phases + i, (uint32_t)sizeof(StepPhase), &desc_bar[i]);
        }
    }
    if (warp == kIssuerWarp0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&pipe.tmem)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    asm volatile("bar.sync 3, %0;\n" ::"n"(kUmmaThreads) : "memory");  // the only barrier the producer warp joins
    tc_fence_after();

    if (warp >= kLoaderWarp0) {
        if (s.num_gemv > 0) load_stages(&pipe, work, s.num_gemv, s.num_slots, s.T, slots, s.status, threadIdx.x - kLoaderWarp0 * 32);
        return;
    }

    bool alive = true;

#pragma unroll 1
    for (int ph = 0; alive && ph < s.num_phases; ++ph) {
        gs.phase = ph;
        if (threadIdx.x == 0) {
            uint32_t polls = 0;
            while (!mbar_try_wait(&desc_bar[ph & 1], (uint32_t)(ph >> 1) & 1u)) {
                if (++polls >= kStepSpinLimit) {
                    abort_flag = 1;
                    atomicExch(s.status, (int32_t)WRK_ERR_TIMEOUT);
                    break;
                }
            }
        }
        WRK_CTA_SYNC();
        if (abort_flag != 0 || pipe.abort_flag != 0) break;
        for (uint32_t polls = 0; polls < 1024 && !mbar_try_wait(&desc_bar[ph & 1], (uint32_t)(ph >> 1) & 1u); ++polls) {}
        const StepPhase& d = desc[ph & 1];
        if (d.type == PH_GEMV) {
            const GemvCore& a = d.gemv;
            UmmaWork wk{};
            if (d.gemv_index >= 0) wk = work[d.gemv_index];
            const int pro_kind = a.prologue;
            const uint32_t T = a.T;
            const uint32_t xp = a.C + 8;
            __half* lnrow = xs;
            __half* xgen = pro_kind == PRO_LN ? xs : xs + (size_t)T * xp;
            const uint32_t pro_rows = pro_kind == PRO_LN ? T : pro_kind == PRO_LN_SHIFT1 ? 2 * T : 3 * T;
            __half* pbias = xs + (size_t)pro_rows * xp;
            const bool any_work = wk.r0 < wk.r1;
            const bool pro = pro_kind != PRO_NONE && (any_work || blockIdx.x == 0);
            // one token and a row that fits one pass of the CTA: the prologue runs in registers
            const bool fast = pro_kind != PRO_NONE && T == 1 && a.C % 128 == 0 && a.C <= (uint32_t)kFastMaxC;
            const int nv = pro_kind == PRO_LN ? 0 : pro_kind == PRO_LN_SHIFT1 ? 1 : 2;
            FastParams fp;
            uint4 wdirect[2];
            if (fast) {
                if (pro) fast_prologue_load(a, nv, fp);
                if (any_work && wk.direct) {
                    // the rows of a `direct` range (at most two) against the prologue's vector, from registers
                    const uint32_t c0 = threadIdx.x * 8;
                    for (int r = 0; r < 2; ++r)
                        if (c0 < a.C && wk.r0 + r < wk.r1)
                            wdirect[r] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(wk.w) + (size_t)(wk.r0 + r) * wk.K + c0);
                }
            } else if (pro_kind != PRO_NONE) {
                // parameters of the prologue: in flight while the CTA waits for the previous phase
                if (pro) {
                    if (pro_kind == PRO_LN) stage_prologue_params<PRO_LN>(a, xgen, xp, lnrow, pbias);
                    else if (pro_kind == PRO_LN_SHIFT1) stage_prologue_params<PRO_LN_SHIFT1>(a, xgen, xp, lnrow, pbias);
                    else stage_prologue_params<PRO_LN_SHIFT2>(a, xgen, xp, lnrow, pbias);
                }
                cp_async_commit();
            }
            alive = gs.wait();
            if (!alive) break;
            if (fast) {
                if (pro) {
                    float xv[2][8];
                    fast_prologue_run(a, nv, fp, scratch, xv);
                    if (any_work) {
                        const GemvProblem& p = a.p[wk.problem];
                        const int sel = nv == 0 ? 0 : p.x_sel;
                        const bool active = threadIdx.x * 8 < a.C;
                        if (wk.direct) {
                            for (int r = 0; r < 2; ++r) {
                                float dot = 0.f;
                                if (active && wk.r0 + r < wk.r1) {
                                    const __half2* h = reinterpret_cast<const __half2*>(&wdirect[r]);
#pragma unroll
                                    for (int e = 0; e < 4; ++e) {
                                        const float2 f = __half22float2(h[e]);
                                        dot = fmaf(f.x, sel == 0 ? xv[0][2 * e] : xv[1][2 * e], dot);
                                        dot = fmaf(f.y, sel == 0 ? xv[0][2 * e + 1] : xv[1][2 * e + 1], dot);
                                    }
                                }
                                if (wk.r0 + r < wk.r1) {  // the same for every thread
                                    const float total = block_sum_256(dot, scratch + (r & 1) * kWarps);
                                    if (threadIdx.x == 0) {
                                        const EpiOperands eo = epilogue_fetch_rt(a.epilogue, a, p, (uint32_t)(wk.r0 + r), 0);
                                        epilogue_one_rt(a.epilogue, a, p, (uint32_t)(wk.r0 + r), 0, total, eo);
                                    }
                                }
                            }
                        } else {
                            const Tile t0 = tile_of(wk, 0, T);
                            fast_stage(sel == 0 ? xv[0] : xv[1], active, wk.kind == MAT_INT8, t0.Q, t0.atom, breg, bconst);
                        }
                    }
                }
            } else if (pro) {
                cp_async_wait<0>();
                if (pro_kind == PRO_LN) run_prologue<PRO_LN>(a, xgen, xp, lnrow, pbias, scratch);
                else if (pro_kind == PRO_LN_SHIFT1) run_prologue<PRO_LN_SHIFT1>(a, xgen, xp, lnrow, pbias, scratch);
                else run_prologue<PRO_LN_SHIFT2>(a, xgen, xp, lnrow, pbias, scratch);
            }
            if (any_work && !wk.direct) {
                const GemvProblem& p = a.p[wk.problem];
                const __half* x = p.x != nullptr ? p.x : xgen + (size_t)p.x_sel * T * xp;
                const uint32_t x_stride = p.x != nullptr ? p.x_stride : xp;
                const bool i8 = wk.kind == MAT_INT8;
                // the operand has one layout per row range (that of its first tile's packing)
                const Tile t0 = tile_of(wk, 0, T);
                if (!fast) {
                    if (i8) digitize(x, x_stride, T, wk.K, t0.Q, t0.atom, breg, bconst, s.nkb_max);
                    else stage_fp16(x, x_stride, T, wk.K, t0.Q, t0.atom, breg);
                }
                if (threadIdx.x == 0) pipe.stage_end = pipe.stage_base + (uint32_t)stages_of(wk, T);
                fence_async_smem();  // the tensor cores read the operand through the async proxy
                WRK_CTA_SYNC();
                if (warp >= kIssuerWarp0 && warp < kIssuerWarp0 + kIssuers) {
                    if (lane == 0) {
                        if (i8) issue_mmas<true>(&pipe, wk, T, s.num_slots, slots, breg, warp - kIssuerWarp0, s.status);
                        else issue_mmas<false>(&pipe, wk, T, s.num_slots, slots, breg, warp - kIssuerWarp0, s.status);
                    }
                } else if (warp < 4) {
                    if (i8) drain_accumulators<true>(&pipe, a, wk, bconst, s.nkb_max, part, s.status);
                    else drain_accumulators<false>(&pipe, a, wk, bconst, s.nkb_max, part, s.status);
                } else if (i8 && warp < 4 + 4 * kDrainGroups) {
                    drain_accumulators<true>(&pipe, a, wk, bconst, s.nkb_max, part, s.status);
                }
                WRK_CTA_SYNC();
                if (threadIdx.x == 0) {
                    if (i8) pipe.i8_base += pipe.stage_end - pipe.stage_base;
                    else pipe.f16_tiles += (uint32_t)((wk.r1 - wk.r0 + 127) / 128);
                    pipe.stage_base = pipe.stage_end;
                }
            }
        } else if (d.type == PH_TMIX) {
            alive = tmix_phase(gs, d.tmix, reinterpret_cast<__half*>(breg));
        } else {
            alive = wkv_phase(gs, d.wkv, reinterpret_cast<__half*>(breg));
        }
        if (!alive) break;
        if (ph + 1 < s.num_phases) {
            gs.arrive();
            if (pipe.abort_flag != 0) break;  // read after the barrier inside arrive(): the same for every thread
            if (threadIdx.x == 0 && ph + 2 < s.num_phases) {
                fence_async_smem();
                mbar_expect_tx(&desc_bar[ph & 1], (uint32_t)sizeof(StepPhase));
                bulk_load(&desc[ph & 1], s.phases + ph + 2, (uint32_t)sizeof(StepPhase), &desc_bar[ph & 1]);
            }
        } else {
            gs.stamp(1);
        }
    }
    cp_async_wait<0>();
    tc_fence_before();
    WRK_CTA_SYNC();
    if (threadIdx.x == 0) {
        // nothing of this CTA may be in flight when it leaves: the loaders stop at the flag (a job that stopped
        // early) and leave with their copies landed; the wait for them is bounded
        pipe.abort_flag = 1;
        if (s.num_gemv > 0)
            for (uint32_t i = 0; i < kStepSpinLimit && *reinterpret_cast<volatile uint32_t*>(&pipe.loaders_done) < (uint32_t)kLoaders; ++i) {}
    }
    WRK_CTA_SYNC();
    if (warp == kIssuerWarp0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(pipe.tmem), "r"(kTmemCols) : "memory");
    }
}

size_t umma_fixed_smem(const UmmaStepArgs& s) {
    return (size_t)s.b_bytes + (size_t)2 * s.nkb_max * sizeof(float2) + (size_t)kDrainGroups * 2 * 128 * sizeof(float) + 1024 /* alignment of the stages */ + 64;
}

constexpr size_t kMaxUmmaSmem = 223 * 1024;  // dynamic; the static arrays (descriptors, barriers) take about 2 KB more

}  // namespace

size_t decode_step_umma_prepare(UmmaStepArgs& s, uint32_t operand_bytes, uint32_t x_bytes, uint32_t kmax_int8) {
    s.nkb_max = std::max<uint32_t>(kmax_int8 / 128, 1);
    s.x_bytes = x_bytes;
    s.b_bytes = (std::max<uint32_t>(operand_bytes, 8192) + 1023) / 1024 * 1024;  // the token-shift / WKV phases use a few KB of it
    s.num_slots = 0;
    const size_t fixed = umma_fixed_smem(s);
    // A multiple of the number of issuers: every slot then has one issuer within a phase, which sees the slot's
    // stages complete in order.  (With any other count an issuer can reach stage g + slots while stage g, another
    // issuer's, is still in flight, and take the parity of g's predecessor for its own stage's.)
    int slots = kMaxSlots;
    while (slots >= kIssuers && fixed + (size_t)slots * kSlotBytes > kMaxUmmaSmem) slots -= kIssuers;
    if (slots < kIssuers) return 0;
    s.num_slots = slots;
    return fixed + (size_t)slots * kSlotBytes;
}

cudaError_t decode_step_umma(const UmmaStepArgs& s, int grid, cudaStream_t stream) {
    static SmemOptIn opt_in;
    if (cudaError_t e = opt_in.ensure(decode_step_umma_kernel, (int)kMaxUmmaSmem); e != cudaSuccess) return e;
    const size_t smem = umma_fixed_smem(s) + (size_t)s.num_slots * kSlotBytes;
    if (s.num_slots < kIssuers || s.num_slots % kIssuers != 0 || s.num_slots > kMaxSlots || smem > kMaxUmmaSmem || s.T > 2)
        return cudaErrorInvalidValue;
    if (cudaError_t e = cudaMemsetAsync(s.barrier, 0, sizeof(uint32_t), stream); e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kUmmaThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, decode_step_umma_kernel, s);
}

}  // namespace k
}  // namespace wrk
