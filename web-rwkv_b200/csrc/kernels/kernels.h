// Launchers of the sm_100a kernels.  Host code calls only these; each returns the launch status.
#pragma once

#include "../common.h"

namespace wrk {
namespace k {

enum MatKind { MAT_FP16 = 0, MAT_INT8 = 1, MAT_NF4 = 2 };

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to a (kernel, device) pair: one of these per kernel,
// asked before every launch, opts the current device in the first time it is seen there.  Devices past the
// mask's width are opted in on every launch (the call is idempotent).
struct SmemOptIn {
    std::atomic<uint64_t> devices{0};
    template <typename Kernel>
    cudaError_t ensure(Kernel kernel, int bytes) {
        int device = 0;
        cudaError_t e = cudaGetDevice(&device);
        if (e != cudaSuccess) return e;
        const uint64_t bit = device >= 0 && device < 64 ? 1ull << device : 0;
        if (bit != 0 && (devices.load(std::memory_order_acquire) & bit) != 0) return cudaSuccess;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e == cudaSuccess && bit != 0) devices.fetch_or(bit, std::memory_order_release);
        return e;
    }
};

// ---- quantizers (quant.cu) -------------------------------------------------------------
cudaError_t quantize_int8(const __half* input, size_t len, __half* minmax, uint8_t* output, int num_sms,
                          cudaStream_t stream);
cudaError_t quantize_nf4(const __half* input, size_t len, const float* table, bool table_sorted, __half* absmax,
                         uint8_t* output, int num_sms, cudaStream_t stream);

// ---- quantized / fp16 matmul (matmul.cu) --------------------------------------------------
struct MatmulArgs {
    int kind;              // MatKind
    const void* matrix;    // [K (or K/2 bytes), M, B] row-major rows
    const __half* scale;   // Int8: (min, max) per 128 flat elements; NF4: absmax per 64; else null
    const float* table;    // NF4: 16 floats on the device
    uint32_t K, M, B;
    uint32_t N;            // tokens
    DView in;              // [K, N, B]
    DView out;             // [M, N, B]
    int act;
    int32_t* status;       // device status word (bounded waits report here); may be null
};
cudaError_t matmul(const MatmulArgs& a, int num_sms, cudaStream_t stream);
// fp16 matrices with K <= 256 (the low-rank adapters' second matrices) at any token count (gemm_small.cu).
bool matmul_small_supported(const MatmulArgs& a);
cudaError_t matmul_small(const MatmulArgs& a, int num_sms, cudaStream_t stream);
// Tensor-memory (tcgen05) GEMM for N >= 16 tokens (gemm_umma.cu).
bool matmul_umma_supported(const MatmulArgs& a);
cudaError_t matmul_umma(const MatmulArgs& a, int32_t* status, cudaStream_t stream);
// Up to four matrices of one weight format, K and token count (each with its own activations, output and activation
// function) as the row tiles of one launch.
bool matmul_umma_group_supported(const MatmulArgs* a, int count);
cudaError_t matmul_umma_group(const MatmulArgs* a, int count, int32_t* status, cudaStream_t stream);

// ---- one-shot all-reduce over peer memory (peer_reduce.cu) --------------------------------------------
constexpr int kMaxPeers = 8;
struct PeerReduceArgs {
    void* regions[kMaxPeers];  // every rank's exchange region ([slot 0][slot 1][flags: one u32 per rank]); [rank] is local
    uint32_t world, rank, slot;
    size_t slot_bytes;
    size_t count;              // f32 elements to add, a multiple of 4
    void* dst;                 // local destination, f16 or f32
    int dst_dtype;
    uint32_t* epoch;           // local: sequence number of the last finished call
    uint32_t* done;            // local: CTAs of the running call that have finished
    int32_t* status;
};
cudaError_t peer_all_reduce(const PeerReduceArgs& a, int num_sms, cudaStream_t stream);

// ---- WKV recurrences (wkv.cu) ------------------------------------------------------------
struct WkvArgs {
    const uint32_t* cursors;  // packed [T] or wide [3 * T]
    int wide;
    DView state;              // f32 [C, S + 1, B]
    uint32_t S, H, T, B;
    int dtype;                // dtype of k, v, r, x (v5/v6) or r, w, n, x (v7)
    const float* time_decay;  // v5: [S, H]; v6: [S, H, T]
    const float* time_first;  // v5/v6: [S, H]
    int per_token_decay;      // v6 = 1, v5 = 0
    const void* k;            // v5/v6
    const void* v;
    const void* r;            // all
    const void* w;            // v7 raw decay
    const void* n;            // v7 stacked k, v, a, kk: [S, H, T, 4]
    void* x;
    int32_t* status;          // device status word
};
cudaError_t time_mix_v56(const WkvArgs& a, cudaStream_t stream);
bool time_mix_v56_chunked_supported(const WkvArgs& a);
cudaError_t time_mix_v56_chunked(const WkvArgs& a, cudaStream_t stream);
cudaError_t time_mix_v7(const WkvArgs& a, cudaStream_t stream);
cudaError_t time_mix_v4(const uint32_t* cursors, int wide, const float* time_decay, const float* time_first, DView state,
                        int dtype, const void* k, const void* v, const void* r, void* x, uint32_t C, uint32_t T,
                        cudaStream_t stream);
cudaError_t time_first_v7(const __half* u, int dtype, const void* r, const void* n, void* x, uint32_t S,
                          uint32_t H, uint32_t T, cudaStream_t stream);

// ---- supporting ops (support.cu) -----------------------------------------------------------
cudaError_t layer_norm(const __half* w, const __half* b, int dtype, void* x, uint32_t C, uint32_t rows,
                       uint32_t wrows, float eps, cudaStream_t stream);
cudaError_t layer_norm_copy(const __half* w, const __half* b, int dtype, const void* delta, void* src, void* x, uint32_t C,
                            uint32_t rows, uint32_t wrows, float eps, cudaStream_t stream);
cudaError_t l2_norm(int dtype, void* x, uint32_t C, uint32_t rows, float eps, cudaStream_t stream);
cudaError_t softmax(int dtype, void* x, uint32_t C, uint32_t rows, cudaStream_t stream);
cudaError_t recenter(int dtype, void* x, uint32_t C, uint32_t rows, cudaStream_t stream);
cudaError_t rms_norm(const __half* w, const __half* b, int dtype, void* x, uint32_t C, uint32_t rows, float eps,
                     cudaStream_t stream);
cudaError_t embed(const uint32_t* tokens, const __half* input, int dtype, void* output, uint32_t C, uint32_t rows,
                  uint32_t vocab, int32_t* status, cudaStream_t stream);
cudaError_t broadcast(DView input, DView output, cudaStream_t stream);
cudaError_t blend(const float* factor, DView input, DView output, cudaStream_t stream);
cudaError_t blend_lora(const float* factor, DView xa, DView xb, DView output, uint32_t K, cudaStream_t stream);
cudaError_t token_shift(const uint32_t* cursors, int wide, DView time_mix, DView state, DView input, DView output,
                        int reversed, cudaStream_t stream);
constexpr uint32_t kShiftMultiMax = 6;
struct ShiftMultiArgs {
    const uint32_t* cursors;
    int wide;
    DView state;          // f32, row 0 = the shift row
    const __half* in;     // [C, T]
    uint32_t C, T, count;
    const __half* mix[kShiftMultiMax];  // [C] each
    __half* out[kShiftMultiMax];        // [C, T] each
    int reversed;
};
cudaError_t token_shift_multi(const ShiftMultiArgs& a, cudaStream_t stream);
// Vector forms for dense operands (elementwise.cu); false: the operands do not fit, nothing was launched.
bool layer_norm_vec(const __half* w, const __half* b, int dtype, const void* delta, void* src, void* x, uint32_t C, uint32_t rows,
                    uint32_t wrows, float eps, cudaStream_t stream);
bool binary_vec(int is_mul, const DView& input, const DView& output, int act_x, int act_y, int act_out, cudaStream_t stream);
bool activate_vec(const DView& x, int act, cudaStream_t stream);
bool blit_vec(const DView& input, const DView& output, cudaStream_t stream);
// `bias`: null, or one row [C, 1, Z] added to the factors first (the sum rounded to f16, as a separate add stores it)
bool token_shift_vec(const uint32_t* cursors, int wide, const DView& time_mix, const DView* bias, const DView& state,
                     const DView& input, const DView& output, int reversed, cudaStream_t stream);
bool token_shift_vec_fits(const DView& time_mix, const DView* bias, const DView& state, const DView& input, const DView& output);
bool token_shift_multi_vec(const ShiftMultiArgs& a, cudaStream_t stream);
// `xres`: null, or the residual stream, which takes xres + x as well
bool channel_mix_vec(const uint32_t* cursors, int wide, const DView& state, int dtype, const void* r, const void* v, void* x,
                     void* xres, uint32_t C, uint32_t T, int v7, cudaStream_t stream);
// group norm of rows of C <= 256 values + copy into f16 + out <- act(gate) * that, in one pass (x is left as it was)
bool group_norm_gate_supported(const __half* w, const __half* b, const void* x, const __half* gate, const __half* out, uint32_t C);
cudaError_t group_norm_gate(const __half* w, const __half* b, int dtype, void* x, uint32_t C, uint32_t rows, uint32_t wrows, float eps,
                            const __half* gate, __half* out, int gate_act, cudaStream_t stream);
struct PackV7Args {
    const __half *k_k, *k_a;  // [H * S]
    __half *k, *kk, *n;       // [S, H, T] (k updated in place), [S, H, T], [S, H, T, 4]
    const __half *v, *a;      // [S, H, T]
    uint32_t S, H, rows;      // rows = H * T
    float eps;
};
cudaError_t pack_v7(const PackV7Args& p, cudaStream_t stream);
cudaError_t shift_carry(const uint32_t* cursors, int wide, DView state, int dtype, const void* x, uint32_t C, uint32_t T,
                        cudaStream_t stream);
cudaError_t channel_mix(const uint32_t* cursors, int wide, DView state, int dtype, const void* r, const void* v,
                        void* x, uint32_t C, uint32_t T, int v7, cudaStream_t stream);
cudaError_t binary(int is_mul, DView input, DView output, int act_x, int act_y, int act_out, cudaStream_t stream);
cudaError_t activate(DView x, int act, cudaStream_t stream);
cudaError_t blit(DView input, DView output, int transpose, cudaStream_t stream);
cudaError_t lerp(DView input, DView output, DView factor, int reversed, cudaStream_t stream);
cudaError_t affine(int dtype, void* x, size_t len, float scale, float bias, cudaStream_t stream);
cudaError_t control_k_v7(const __half* p, DView a, DView k, cudaStream_t stream);

}  // namespace k
}  // namespace wrk
