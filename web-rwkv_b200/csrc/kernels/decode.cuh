// Fused decode path (few tokens per job): argument blocks of the kernels in decode.cu.
#pragma once

#include "kernels.h"

namespace wrk {
namespace k {

constexpr int kMaxProblems = 5;
constexpr int kDecodeMaxTokens = 8;  // one MMA n-tile

// One weight matrix of a grouped weight-streaming launch: out[t][m] = epilogue(act(W[m,:] . x[t,:])).
struct GemvProblem {
    const uint8_t* w;      // rows of K elements (fp16: 2K bytes, Int8: K bytes, NF4: K/2 bytes)
    const __half* scale;   // Int8 (min, max) per 128; NF4 absmax per 64; fp16: null
    int32_t kind;          // MatKind
    uint32_t K, M;
    const __half* x;       // [T] rows of K fp16, x_stride elements apart; null = take prologue vector x_sel
    int32_t x_sel;
    uint32_t x_stride;
    void* out;             // [T] rows of M, out_stride elements apart
    uint32_t out_stride;
    int32_t out_dtype;
    int32_t act;
};

enum GemvPrologue { PRO_NONE = 0, PRO_LN = 1, PRO_LN_SHIFT1 = 2, PRO_LN_SHIFT2 = 3 };
enum GemvEpilogue { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_CHANNEL_MIX = 2 };

// Row range of one problem handled by a CTA.
struct GemvSegment {
    int32_t problem, row0, row1, pad;
};
constexpr int kSegmentsPerCta = 3;
constexpr int kInlineCtas = 192;

// What the device math of a weight-streaming launch (or phase) needs: the matrices, the prologue and the epilogue.
struct GemvCore {
    GemvProblem p[kMaxProblems];
    int32_t num_problems;
    uint32_t kmax;                // largest K of the launch (filled in by fused_gemv)
    uint32_t T;
    const float* table;           // NF4 code book (device)
    int32_t* status;
    // prologue: layer norm of `ln_x` (+ token shift against the carry row `state`)
    int32_t prologue;
    const __half* ln_x;           // rows of C fp16; prologue row t reads row t + ln_row_off[t]
    int32_t ln_row_off[kDecodeMaxTokens];
    const __half* ln_w;
    const __half* ln_b;
    float ln_eps;
    uint32_t C;
    const uint32_t* cursors;
    int32_t wide;
    DView state;                  // f32 carry row (row 0 of the view)
    const __half* mix0;           // [C] token-shift factors of prologue vector 0 / 1
    const __half* mix1;
    int32_t reversed;
    __half* ln_out;               // [T][C] normalised rows, written by CTA 0 (null = skip)
    // epilogue
    int32_t epilogue;
    __half* xres;                 // [T][M] residual stream updated in place
    const __half* cm_r;           // channel mix: receptance [T][M]
    const __half* cm_x;           // channel mix: normalised ffn input [T][M] (becomes the carry row)
    DView cm_state;
    float rescale;                // 1.0 or 0.5 applied to the residual stream after the add
};

struct FusedGemvArgs : GemvCore {
    int32_t ring_depth;           // staging cells per warp (filled in by fused_gemv)
    const GemvSegment* segments;  // [grid][kSegmentsPerCta], row0 == row1 marks an unused entry
    // The same partition as boundaries in the concatenated row space of the launch's matrices (filled in by
    // fused_gemv for grids of at most kInlineCtas): CTA c owns rows [cta_row_start[c], cta_row_start[c + 1]).
    // Read from the kernel parameters, it spares every CTA a dependent global load before its first copy.
    int32_t inline_partition;
    uint32_t cta_row_start[kInlineCtas + 1];
};

cudaError_t fused_gemv(const FusedGemvArgs& a, int grid, cudaStream_t stream);
bool fused_gemv_partition(const FusedGemvArgs& a, int grid, std::vector<GemvSegment>& table);
// Copies the partition's boundaries into the launch arguments (grids of at most kInlineCtas).
void fused_gemv_inline_partition(FusedGemvArgs& a, int grid, const std::vector<GemvSegment>& table);
// Dynamic shared memory of a launch with `depth` staging cells per warp (clamped to the supported 2 .. 4).
size_t fused_gemv_smem(uint32_t T, uint32_t Kmax, uint32_t C, int prologue, int depth);

// v6 data-dependent token shift: time_mix_w2 (5 x [D -> C]) + static mixes + 5-way shift.
struct TmixArgs {
    const __half* w2;        // [5][C][D] fp16
    const __half* tmx;       // [T][5 * D] fp16 (tanh'ed adapter activations)
    const __half* mix;       // [5][C] static mixes
    const __half* att_x;     // [T][C] normalised input
    const uint32_t* cursors;
    int32_t wide;
    DView state;             // carry row
    __half* sx;              // [5][T][C]
    uint32_t C, D, T;
};
cudaError_t tmix_shift_v6(const TmixArgs& a, cudaStream_t stream);

// v5 / v6 time-mix block: decay adapter (v6), WKV recurrence, group norm, gate.
struct Wkv6Args {
    const uint32_t* cursors;
    int32_t wide;
    DView state;             // f32 [C, S + 1, B]
    uint32_t H, T, B;
    int32_t per_token_decay; // v6
    const __half* tdw;       // v6: [T][D] tanh'ed decay adapter activations
    const __half* td_w2;     // v6: [C][D] fp16
    const __half* td0;       // v6: [C] fp16 static decay
    const float* td5;        // v5: [C] f32 decay, already exp(-exp(.))
    uint32_t D;
    const float* time_first; // [C]
    const float* k;          // [T][C] f32
    const float* v;
    const float* r;
    const __half* g;         // [T][C] fp16 gate pre-activation
    const __half* att_x;     // [T][C] normalised input (carry source)
    const __half* gn_w;      // [C]
    const __half* gn_b;
    float gn_eps;
    __half* out;             // [T][C] gated output
};
cudaError_t wkv56_fused(const Wkv6Args& a, cudaStream_t stream);

// Int8 GEMV (y[t][m] = act(W[m][:] . x[t][:]), f16 x, f32 y) whose row-range table lives in a static
// device array of kStaticGemvMaxCtas ranges: neither the first call on a device (which looks the array up)
// nor any later one allocates.  `device` must be the current device.  Returns a StaticGemvError.
constexpr int kStaticGemvMaxCtas = 512;
constexpr int kStaticGemvMaxDevices = 64;
enum StaticGemvError { SG_OK = 0, SG_TOO_MANY_CTAS = 1, SG_BAD_SHAPE = 2, SG_BAD_DEVICE = 3, SG_CUDA = 4 };
int gemv_int8_static(int device, cudaStream_t stream, const uint8_t* w, const __half* minmax, const __half* x, float* y,
                     uint32_t K, uint32_t M, uint32_t T, int act, uint32_t num_ctas, cudaError_t* cuda_error);

// ---- the whole decode step in one persistent kernel (decode_step.cu) -----------------------------------
// A job of a few tokens runs as a list of phases inside one cooperative launch of one CTA per SM; the CTAs meet
// at a grid-wide barrier between phases.  A CTA's copies of weights run ahead of its math across phase
// boundaries (weights never change during a job), so the stream of weights does not stop while a barrier, a
// layer norm or the WKV recurrence is in progress.
enum StepPhaseType { PH_GEMV = 0, PH_TMIX = 1, PH_WKV = 2 };

struct alignas(16) StepPhase {
    int32_t type;
    int32_t gemv_index;  // PH_GEMV: index into the CTA's work list, -1 for a phase without matrices
    union {
        GemvCore gemv;
        TmixArgs tmix;
        Wkv6Args wkv;
    };
};
static_assert(sizeof(StepPhase) % 16 == 0, "phases are fetched with 16-byte bulk copies");

// One CTA's share of one weight-streaming phase: rows [r0, r1) of one matrix (r0 == r1: none).
struct StepWork {
    const uint8_t* w;
    const __half* scale;
    int32_t r0, r1;
    uint32_t K;
    int16_t kind, problem;
};
static_assert(sizeof(StepWork) == 32, "work lists are fetched with 16-byte bulk copies");

struct StepArgs {
    const StepPhase* phases;
    int32_t num_phases;
    const StepWork* work;     // [grid][num_gemv]
    int32_t num_gemv;
    uint32_t T;               // tokens of the job (the largest T of any phase)
    uint32_t kmax;            // largest K of any matrix
    uint32_t C;
    int32_t ring_depth;
    uint32_t x_halfs;         // fp16 elements reserved for staged activations / prologue rows
    const float* table;       // NF4 code book or null
    uint32_t* barrier;        // grid barrier counter; the launcher zeroes it on the stream before the kernel
    int32_t* status;          // device status word: a wait that gives up writes WRK_ERR_TIMEOUT here
    unsigned long long* timeline;  // optional [2 * num_phases][grid] globaltimer stamps (phase start / end)
};
// Shared memory of the step kernel for a job shape, or 0 when it does not fit; fills ring_depth and x_halfs.
size_t decode_step_prepare(StepArgs& s, bool any_prologue);
cudaError_t decode_step(const StepArgs& s, int grid, cudaStream_t stream);

// ---- the same job with the matrices on the 5th-generation tensor cores (decode_step_umma.cu) ----------------
// Int8 and fp16 matrices, jobs of one or two tokens.  A CTA's rows of a matrix arrive as blocks of
// [rows][128 bytes] in a ring of 16 KB stages (cp.async by four loader warps, into the 128-byte-swizzled operand
// layout) and are multiplied straight from shared memory by tcgen05.mma (kind::i8 against the activations as three
// signed-byte digits per value, kind::f16 against fp16 activations); the accumulators live in tensor memory.
struct UmmaWork {
    const uint8_t* w;       // the matrix: rows of K bytes (Int8) or 2 K bytes (fp16)
    const __half* scale;    // Int8: (min, max) per 128 weights
    int32_t r0, r1;         // rows [r0, r1) of the matrix (r0 == r1: none)
    uint32_t K;
    int16_t kind, problem;
    int32_t direct;         // 1: a few rows of an fp16 matrix fed by a one-token prologue: multiplied from registers,
                            // never staged (the loaders and issuers skip the entry)
    uint8_t pad_[28];
};
static_assert(sizeof(UmmaWork) == 64, "work lists are fetched with 16-byte bulk copies");

// Geometry of one 128-row tile of a CTA's row range: P stage rows per k-block, Q k-blocks per stage; a stage's
// activation operand is one 8-row atom (Q == 1) or two.
struct UmmaTile {
    int rows, P, Q, nkb, nslots;
    uint32_t xstep;  // elements of the tensor map per k-block (128 bytes)
    uint32_t atom;   // bytes of the activation operand per stage
};
__host__ __device__ inline UmmaTile umma_tile(int total_rows, int tile, int kind, uint32_t K, uint32_t T) {
    UmmaTile t;
    const bool i8 = kind == MAT_INT8;
    const int left = total_rows - tile * 128;
    t.rows = left < 128 ? left : 128;
    // the blocks of a stage share one MMA: block i's activations take columns [i * c, (i + 1) * c) of its 16
    const int cols = i8 ? 3 * (int)T : (int)T;
    int q = t.rows <= 32 ? 4 : t.rows <= 64 ? 2 : 1;
    if (total_rows > 128) q = 1;  // the operand has one layout per range: ranges of several tiles do not pack their last one
    while (q * cols > 16) q >>= 1;
    t.Q = q;
    t.P = 128 / q;
    // activation rows of a stage: up to eight fit one 8-row atom (1 KB; the MMA's columns 8-15 then alias 0-7)
    t.atom = q * cols > 8 ? 2048u : 1024u;
    t.nkb = i8 ? (int)(K / 128) : (int)(K / 64);
    t.nslots = (t.nkb + t.Q - 1) / t.Q;
    t.xstep = i8 ? 128u : 64u;
    return t;
}
__host__ __device__ inline uint32_t umma_operand_bytes(int total_rows, int kind, uint32_t K, uint32_t T) {
    if (total_rows <= 0) return 0;
    const UmmaTile t = umma_tile(total_rows, 0, kind, K, T);
    return (uint32_t)t.nslots * t.atom;
}

struct UmmaStepArgs {
    const StepPhase* phases;
    int32_t num_phases;
    const UmmaWork* work;   // [grid][num_gemv]
    int32_t num_gemv;
    uint32_t T, C;
    int32_t num_slots;      // 16 KB stages (filled in by decode_step_umma_prepare)
    uint32_t b_bytes;       // activation operand region: 1 KB per k-block of the longest row (+ the prologue rows)
    uint32_t x_bytes;       // prologue rows at the end of that region
    uint32_t nkb_max;       // most 128-weight blocks of any Int8 row
    uint32_t* barrier;
    int32_t* status;
    unsigned long long* timeline;
};
// Shared memory of the kernel for a job shape (0: does not fit); fills num_slots, b_bytes, x_bytes.
// `operand_bytes`: the largest activation operand of any CTA and phase, plus the prologue rows where the phase
// has a prologue (b_bytes); x_bytes: the prologue rows alone.
size_t decode_step_umma_prepare(UmmaStepArgs& s, uint32_t operand_bytes, uint32_t x_bytes, uint32_t kmax_int8);
cudaError_t decode_step_umma(const UmmaStepArgs& s, int grid, cudaStream_t stream);

}  // namespace k
}  // namespace wrk
