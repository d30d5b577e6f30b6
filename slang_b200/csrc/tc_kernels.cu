// Tensor-core (tcgen05 / TMEM / TMA) kernels for sm_100a.
//
// learnGradient for wide networks (16-bit storage, fp32 accumulate): two to five layers, up to 64 inputs,
// hidden widths up to 128, up to 64 outputs, every width zero-padded to the shape
// 64 -> 128 -> ... -> 128 -> 64 that the benchmark network has exactly.  One persistent CTA per SM walks
// 64-sample tiles.  All five weight matrices stay in
// shared memory for the whole launch, every layer product of the forward and backward pass is a
// tcgen05.mma with the accumulator in tensor memory, the weight-gradient products accumulate in
// tensor memory across all of the CTA's tiles, and each parameter receives one atomic add per CTA at
// the end.  Activations never leave the SM.
//
// Orientation: features run along the 128 TMEM lanes (the MMA's M), samples along the columns (N = 64):
//   forward   Z_l^T [out x 64]  = W_l [out x in]   . A_l^T          A: W_l, K-major      B: A_l,  MN-major
//   input     dA_l^T [in x 64]  = W_l^T [in x out] . dZ_l^T         A: W_l, MN-major     B: dZ_l, MN-major
//   weights   dW_l [out x in]  += dZ_l^T [out x 64] . A_l [64 x in]  A: dZ_l, K-major     B: A_l,  K-major
// so a single copy of W_l (row-major rows of 128 bytes, 128-byte swizzle) serves both directions.  The
// hidden activations and their gradients are stored feature-major, [128 features][64 samples] with the
// samples of a feature contiguous (one 128-byte swizzled row per feature): the epilogue thread that owns
// a feature writes its 16 samples as two 16-byte stores, the row is a K-major operand of the weight-
// gradient products (K = samples) and an MN-major operand of the layer products (N = samples).  The input
// tile and the target / dZ_4 tile keep the layout they arrive in, [64 samples][64 features].
// An epilogue thread owns one feature (one TMEM lane) and 32 of the 64 sample columns: the bias is a
// per-thread constant and the bias gradient a per-thread sum.
//
// What the reference does instead: one thread per sample and per-element global atomics
// (examples/mlp-training/mlp_sw.slang:28-58, mlvec_sw.slang:53-64), or one warp per 32 samples on
// mma.sync with a per-workgroup reduction (source/standard-modules/neural/mma-tiled-cuda.slang:88-525).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string>

#include "launchers.h"
#include "mlp_common.cuh"
#include "tc_host.h"
#include "tc_ptx.cuh"

namespace mlpb200 {

using namespace ptx;

// Status-word codes (which wait gave up).
enum : uint32_t {
    kStatusCtrlAcc = 1u, kStatusCtrlX = 2u, kStatusEpiAcc = 4u, kStatusEpiTarget = 8u, kStatusEpiLoss = 16u, kStatusAlign = 32u,
};

// Developer builds (-DMLPB200_TRACE, never the shipped library) record clock64() time stamps of one
// tile's hand-offs in CTA 0 into WideTrainParams::timing; the shipped kernel reads no clock.
#ifdef MLPB200_TRACE
#define MLPB200_TRACE_AT(cond, slot) do { if (cond) p.timing[slot] = (unsigned long long)clock64(); } while (0)
#else
#define MLPB200_TRACE_AT(cond, slot) do { } while (0)
#endif

namespace wide {
constexpr int NS = 64;            // samples per tile
constexpr int CH = 32;            // samples per chain (MMA N of the forward / input-gradient products)
constexpr int NCH = NS / CH;      // chains per tile
constexpr int D0 = 64, H = 128, DOUT = 64;  // padded widths: inputs, hidden layers, outputs
constexpr int kMaxLayers = 5;
constexpr int CPT = 8;            // sample columns of EACH chain per epilogue thread
#ifdef MLPB200_TRACE
constexpr uint32_t kTraceTile = 3;  // which of CTA 0's tiles a trace build records
#endif
constexpr int kEpiWarps = 16;     // 4 TMEM lane quarters x 4 column groups; every warp serves both chains
constexpr int kThreads = 64 + 32 * kEpiWarps;  // warp 0: TMA + MMA issue, warp 1: TMEM owner, then the epilogue warps

// Shared-memory map (bytes from a 1024-aligned base).  Operand buffers are panels of
// [rows][128 bytes] with the 128-byte swizzle; a panel holds 64 16-bit features of every row.
constexpr uint32_t kW0 = 0;                  // 128 rows x 1 panel
constexpr uint32_t kW1 = 16384;              // 128 rows x 2 panels (panel stride 16384)
constexpr uint32_t kW2 = kW1 + 32768;
constexpr uint32_t kW3 = kW2 + 32768;
constexpr uint32_t kW4 = kW3 + 32768;        // 64 rows x 2 panels (panel stride 8192)
constexpr uint32_t kX = kW4 + 16384;         // 2 buffers x [64 rows x 1 panel]
constexpr uint32_t kA1 = kX + 2 * 8192;      // A_1..A_4: [128 feature rows][64 samples] each, 128-byte rows
constexpr uint32_t kDZ4 = kA1 + 4 * 16384;   // [64 rows x 1 panel]: targets land here, dZ_4 replaces them
constexpr uint32_t kBias = kDZ4 + 8192;      // fp32 [5][128]; row 4 holds the output layer's biases whatever the layer count
constexpr uint32_t kLossPart = kBias + 5 * 128 * 4;  // fp32 [8 feature groups][64 samples]
constexpr uint32_t kBars = kLossPart + 8 * 64 * 4;   // mbarriers: x_full[2], t_full, acc_full[2], acc_free[2], out_full, out_free
constexpr uint32_t kTmemPtr = kBars + 12 * 8;
constexpr uint32_t kAbort = kTmemPtr + 4;
constexpr uint32_t kSmemBytes = kAbort + 4;   // the dynamic shared-memory base must be 1024-byte aligned (checked at run time)
static_assert(kSmemBytes <= 232448, "shared-memory map exceeds the per-CTA limit");

// Tensor-memory columns.
constexpr uint32_t kColDW1 = 0, kColDW4T = 384, kColAcc = 448, kTmemCols = 512;

// Layer l of an NL-layer network: layer 0 and the output layer have their own regions, the hidden-to-hidden
// layers take W1..W3 in order (unused regions stay idle for shorter networks).
__host__ __device__ constexpr uint32_t w_off(int l, int NL) { return l == 0 ? kW0 : l == NL - 1 ? kW4 : kW1 + (uint32_t)(l - 1) * 32768u; }
__host__ __device__ constexpr int in_dim(int l) { return l == 0 ? D0 : H; }
__host__ __device__ constexpr int out_dim(int l, int NL) { return l == NL - 1 ? DOUT : H; }
}  // namespace wide

template <int FMT> struct Elem;
template <> struct Elem<MLP_BF16> {
    static constexpr uint32_t kUmmaFmt = 1;
    __device__ static __forceinline__ uint16_t pack(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }
    __device__ static __forceinline__ float unpack(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
    // Round to nearest even with integer operations (keeps the conversion unit free for tanh).
    __device__ static __forceinline__ float round(float v)
    {
        const uint32_t u = __float_as_uint(v);
        return __uint_as_float((u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u);
    }
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi)
    {
        __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&t);
    }
    __device__ static __forceinline__ float unpack_lo(uint32_t p) { return __uint_as_float(p << 16); }
    __device__ static __forceinline__ float unpack_hi(uint32_t p) { return __uint_as_float(p & 0xffff0000u); }
};
template <> struct Elem<MLP_F16> {
    static constexpr uint32_t kUmmaFmt = 0;
    __device__ static __forceinline__ uint16_t pack(float v) { return __half_as_ushort(__float2half_rn(v)); }
    __device__ static __forceinline__ float unpack(uint16_t b) { return __half2float(__ushort_as_half(b)); }
    __device__ static __forceinline__ float round(float v) { return unpack(pack(v)); }
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi)
    {
        __half2 t = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&t);
    }
    __device__ static __forceinline__ float unpack_lo(uint32_t p) { return unpack((uint16_t)(p & 0xffffu)); }
    __device__ static __forceinline__ float unpack_hi(uint32_t p) { return unpack((uint16_t)(p >> 16)); }
};

// Hidden activation on a storage-rounded pre-activation: value and derivative.
template <int ACT>
__device__ __forceinline__ void act_pair(float z, float alpha, float& a, float& d)
{
    if constexpr (ACT == MLP_ACT_GELU_TANH) {
        const float c0 = MLPB200_SQRT_2_OVER_PI, c1 = MLPB200_SQRT_2_OVER_PI * MLPB200_GELU_C;
        const float z2 = z * z;
        const float t = tanh_approx(z * fmaf(c1, z2, c0));
        const float hz = 0.5f * z;
        a = fmaf(hz, t, hz);
        d = fmaf(hz * fmaf(-t, t, 1.0f), fmaf(3.0f * c1, z2, c0), fmaf(0.5f, t, 0.5f));
    } else if constexpr (ACT == MLP_ACT_RELU) {
        a = fmaxf(z, 0.0f);
        d = z > 0.0f ? 1.0f : (z == 0.0f ? 0.5f : 0.0f);
    } else if constexpr (ACT == MLP_ACT_LEAKY_RELU) {
        a = z < 0.0f ? alpha * z : z;
        d = z < 0.0f ? alpha : 1.0f;
    } else {
        a = z;
        d = 1.0f;
    }
}
// Activation chosen at run time (any of the library's activations).
__device__ __forceinline__ void act_pair_rt(int act, float z, float alpha, float& a, float& d)
{
    a = act_value(act, alpha, z);
    d = act_deriv(act, alpha, z);
}

// The same on two samples at once with the packed fp32 instructions of sm_100 (two results per
// issued instruction): the epilogue is bound by instruction issue, not by the arithmetic units.
template <int ACT>
__device__ __forceinline__ void act_pair2(float2 z, float alpha, float2& a, float2& d)
{
    if constexpr (ACT == MLP_ACT_GELU_TANH) {
        const float c0 = MLPB200_SQRT_2_OVER_PI, c1 = MLPB200_SQRT_2_OVER_PI * MLPB200_GELU_C;
        const float2 C0 = make_float2(c0, c0), C1 = make_float2(c1, c1), C3 = make_float2(6.0f * c1, 6.0f * c1), C2 = make_float2(2.0f * c0, 2.0f * c0);
        const float2 HALF = make_float2(0.5f, 0.5f), NHALF = make_float2(-0.5f, -0.5f);
        // With s = (1 + tanh u) / 2 and u = z (c0 + c1 z^2): gelu = z s and, because 1 - tanh^2 = 4 s (1 - s),
        // gelu' = s + z s' = s + (z s) (1 - s) (2 c0 + 6 c1 z^2): nine packed operations and two tanh.
        const float2 z2 = __fmul2_rn(z, z);
        const float2 u = __fmul2_rn(z, __ffma2_rn(C1, z2, C0));
        const float2 t = make_float2(tanh_approx(u.x), tanh_approx(u.y));
        const float2 sg = __ffma2_rn(HALF, t, HALF);
        a = __fmul2_rn(z, sg);
        const float2 om = __ffma2_rn(NHALF, t, HALF);
        const float2 w = __ffma2_rn(C3, z2, C2);
        d = __ffma2_rn(__fmul2_rn(a, om), w, sg);
    } else {
        act_pair<ACT>(z.x, alpha, a.x, d.x);
        act_pair<ACT>(z.y, alpha, a.y, d.y);
    }
}

struct WideTrainParams {
    int dims[wide::kMaxLayers + 1];  // the network's real widths
    int hidden_act;                  // used when the kernel is built for a run-time activation
    int param_layout;                // MlpParamLayout of the weights (forward-only builds read either)
    int storage_dtype;               // MlpDType of parameters and biases in memory; MLP_F32 = fp32 storage with 16-bit
                                     // operands: weights converted at staging, pre-activations and outputs not rounded
    int t_direct;                    // 1: the epilogue reads targets from global memory itself (no tensor map)
    int target_dtype;
    const void* targets;             // for t_direct
    float* outputs;                  // forward-only builds: fp32 [count][outputs]
    const MlpLayerPointers* net;
    uint32_t* loss_words;
    uint32_t* status;
    uint32_t count;
    uint32_t n_tiles;
    float loss_scale;  // 1 / outputs for the mean-squared error, 1 for the sum of squares
    float act_alpha;
    float* input_grads;          // optional (training): fp32 [count][dims[0]] gradient with respect to the inputs
    unsigned long long* timing;  // trace builds only: time stamps written by CTA 0
};

// FWD builds stop after the output layer and write the network outputs (the "forward" entry point of the same
// shapes): no targets, no derivatives, no gradient products.
// F32S: fp32 parameter storage with 16-bit operands (weights converted while they are staged, pre-activations and
// outputs not rounded); such networks run the builds with the activation chosen at run time.
// XTRA: training builds that also write the input gradients (WideTrainParams::input_grads) and / or write the weight
// gradients in the tiled parameter layout; the plain training builds carry neither test (they cost 2.5 % at
// the benchmark shape when they were run-time options of one build).
template <int FMT, int ACT, int NL, bool FWD, bool F32S = false, bool XTRA = false>
__global__ void __launch_bounds__(wide::kThreads, 1)
learn_gradient_wide_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_t,
                           const WideTrainParams p)
{
    using namespace wide;
    using E = Elem<FMT>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    const uint32_t sbase = smem_u32(smem);
    if (sbase & 1023u) {  // the swizzled operand layouts need a 1024-byte aligned base
        if (threadIdx.x == 0) atomicOr(p.status, kStatusAlign);
        return;
    }
    uint64_t* bars = (uint64_t*)(smem + kBars);
    uint64_t* x_full = bars;        // [2]
    uint64_t* t_full = bars + 2;
    uint64_t* acc_full = bars + 3;  // [2], one per chain
    uint64_t* acc_free = bars + 5;  // [2]
    uint64_t* out_full = bars + 7;  // the output layer's accumulator (whole tile) is complete
    uint64_t* out_free = bars + 8;  // ... has been consumed, dZ_4 and the loss terms are in shared memory
    uint32_t* tmem_ptr = (uint32_t*)(smem + kTmemPtr);
    volatile uint32_t* abort_flag = (volatile uint32_t*)(smem + kAbort);
    float* s_bias = (float*)(smem + kBias);
    float* s_loss_part = (float*)(smem + kLossPart);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n_my_tiles = (p.n_tiles > blockIdx.x) ? (p.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    // ---- set-up: barriers, tensor memory, weights and biases into shared memory ------------------
    if (threadIdx.x == 0) {
        mbar_init(&x_full[0], 1);
        mbar_init(&x_full[1], 1);
        mbar_init(t_full, 1);
        for (int h = 0; h < NCH; ++h) {
            mbar_init(&acc_full[h], 1);
            mbar_init(&acc_free[h], kEpiWarps);  // every epilogue warp works on every chain
        }
        mbar_init(out_full, 1);
        mbar_init(out_free, kEpiWarps);
        *abort_flag = 0u;
        fence_mbar_init();
        prefetch_tmap(&tmap_x);
        prefetch_tmap(&tmap_t);
    }
    if (warp == 1) {
        tmem_alloc(tmem_ptr, kTmemCols);
        tmem_relinquish();
    }
    for (int l = 0; l < NL; ++l) {
        // Real widths in x out, padded to inp x outp with zeros (padded rows, columns and biases are zero, so
        // padded features carry no signal forward and receive no gradient).
        const int in = p.dims[l], out = p.dims[l + 1];
        const int inp = in_dim(l), outp = out_dim(l, NL);
        const uint16_t* w16 = (const uint16_t*)p.net[l].weights;
        const float* w32 = (const float*)p.net[l].weights;
        constexpr bool fp32_storage = F32S;
        const int chunks_per_row = inp / 8;  // 16-byte chunks: 8 elements
        const uint32_t panel_stride = (uint32_t)outp * 128u;
        const bool rows_aligned = (in & 7) == 0 && p.param_layout == MLP_PARAMS_ROW_MAJOR && !fp32_storage;
        for (int idx = threadIdx.x; idx < outp * chunks_per_row; idx += kThreads) {
            const int o = idx / chunks_per_row, c = idx % chunks_per_row;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (o < out && c * 8 < in) {
                if (rows_aligned) {
                    v = *(const uint4*)(w16 + (size_t)o * in + c * 8);
                } else {
                    uint16_t hw[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        hw[j] = 0;
                        if (c * 8 + j < in) {
                            const int64_t wi = weight_index(p.param_layout, in, out, o, c * 8 + j);
                            hw[j] = fp32_storage ? E::pack(w32[wi]) : w16[wi];
                        }
                    }
                    v = make_uint4(hw[0] | ((uint32_t)hw[1] << 16), hw[2] | ((uint32_t)hw[3] << 16), hw[4] | ((uint32_t)hw[5] << 16),
                                   hw[6] | ((uint32_t)hw[7] << 16));
                }
            }
            const uint32_t off = w_off(l, NL) + (uint32_t)(c >> 3) * panel_stride + (uint32_t)o * 128u + (uint32_t)(((c & 7) ^ (o & 7)) << 4);
            *(uint4*)(smem + off) = v;
        }
        const int brow = l == NL - 1 ? kMaxLayers - 1 : l;
        for (int j = threadIdx.x; j < 128; j += kThreads)
            s_bias[brow * 128 + j] = j < out ? load_as_f32(F32S ? MLP_F32 : FMT, (const void*)p.net[l].biases, j) : 0.0f;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    if (warp == 0) {
        // =================================== control warp ==========================================
        // The 64 samples of a tile run as two chains of 32 (h = 0, 1) through the hidden layers: while the
        // epilogue warps work on one chain's accumulator, the tensor pipe runs the other chain's product.
        // Both chains share the operand buffers (sample columns 32h..32h+31) and the weight-gradient
        // accumulators.  They meet twice per tile: at the output layer, whose product covers the whole
        // tile with the samples on the TMEM lanes (see the epilogue), and at the dW_0 product.
        // The whole warp walks the schedule (the waits); one elected lane issues the TMA loads, the MMAs
        // and the commits as straight-line code: the fewer instructions this warp needs per product, the
        // less its issue rate suffers from the four busy epilogue warps on its scheduler.
        if (n_my_tiles > 0) {
            const bool leader = elect_one();
            constexpr uint32_t F = E::kUmmaFmt;
            constexpr uint32_t kIdescFwd0 = umma_idesc(F, 0, 0, 128, CH);   // W_0 (K) x input tile (K)
            constexpr uint32_t kIdescFwd = umma_idesc(F, 0, 1, 128, CH);    // W (K) x act (MN: samples contiguous)
            constexpr uint32_t kIdescOut = umma_idesc(F, 1, 0, 128, 64);    // A_4 (MN: samples on the lanes) x W_4 (K)
            constexpr uint32_t kIdescDx4 = umma_idesc(F, 1, 0, 128, CH);    // W_4^T (MN) x dZ_4 (K: features contiguous)
            constexpr uint32_t kIdescDx = umma_idesc(F, 1, 1, 128, CH);     // W^T (MN) x dZ (MN)
            constexpr uint32_t kIdescDw = umma_idesc(F, 0, 0, 128, 128);    // dZ (K = samples) x act (K = samples)
            constexpr uint32_t kIdescDw64 = umma_idesc(F, 0, 1, 128, 64);   // act or dZ_0 (K) x dZ_4 or input tile (MN)
            uint32_t n_free0 = 0, n_free1 = 0;  // phases of acc_free[h] this warp has consumed
            bool ok = true;
#ifdef MLPB200_TRACE
            bool tr_on = false;  // this lane records the traced tile
            uint32_t tr_step = 0;
#endif
            // Every phase of a barrier is observed in order: a parity wait only means something if
            // the waiter has seen all earlier phases complete.
            auto chain_wait = [&](int h) {
                MLPB200_TRACE_AT(tr_on, (tr_step * 2 + h) * 3 + 0);
                uint32_t& n = h == 0 ? n_free0 : n_free1;
                ok = ok && mbar_wait(&acc_free[h], n & 1u, abort_flag, p.status, kStatusCtrlAcc);
                ++n;
                tc_fence_after();
                MLPB200_TRACE_AT(tr_on, (tr_step * 2 + h) * 3 + 1);
            };
            // Descriptors cost one 32-bit add each: the high word (8-row groups 1024 bytes apart,
            // version 1, 128-byte swizzle) is the same for every operand and the low word is the
            // buffer's address in 16-byte units plus compile-time offsets.
            const uint32_t lo_base = (sbase & 0x3FFFFu) >> 4;
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            // K-major operand: rows of 128 bytes; a K step of 16 elements is 32 bytes inside the
            // swizzled row; 64-element panels are `panel` bytes apart.
            auto desc_k = [&](uint32_t buf, uint32_t panel, int k) -> uint64_t {
                const uint32_t lo = lo_base + ((buf + (uint32_t)(k >> 2) * panel + (uint32_t)(k & 3) * 32u) >> 4) + (1u << 16);
                return ((uint64_t)kDescHi << 32) | lo;
            };
            // MN-major operand: a K step of 16 rows is 2048 bytes; 64-element panels are `panel` bytes apart.
            auto desc_mn = [&](uint32_t buf, uint32_t panel, int k) -> uint64_t {
                const uint32_t lo = lo_base + ((buf + (uint32_t)k * 2048u) >> 4) + ((panel >> 4) << 16);
                return ((uint64_t)kDescHi << 32) | lo;
            };
            if (leader) {
                mbar_expect_tx(&x_full[0], 8192);
                tma_load_2d(smem + kX, &tmap_x, 0, (int32_t)(blockIdx.x * NS), &x_full[0]);
                if (!p.t_direct) {
                    mbar_expect_tx(t_full, 8192);
                    tma_load_2d(smem + kDZ4, &tmap_t, 0, (int32_t)(blockIdx.x * NS), t_full);
                }
            }
            uint32_t loads_issued = 1;  // tiles whose X and target loads have been issued (for the drain after an abort)

            for (uint32_t it = 0; it < n_my_tiles && ok; ++it) {
                const uint32_t b = it & 1u;
                const uint32_t next_tile = blockIdx.x + (it + 1) * gridDim.x;
                const bool has_next = it + 1 < n_my_tiles;
                const uint32_t xbuf = kX + b * 8192u;
#ifdef MLPB200_TRACE
                tr_on = leader && blockIdx.x == 0 && it == kTraceTile && p.timing;
                tr_step = 0;
#endif
                // ---- forward, layer 0 ----
#pragma unroll
                for (int h = 0; h < NCH; ++h) {
                    if constexpr (FWD) {
                        // the previous tile's outputs have left the accumulator
                        if (h == 0 && it > 0) {
                            ok = ok && mbar_wait(out_free, (it - 1) & 1u, abort_flag, p.status, kStatusCtrlAcc);
                            tc_fence_after();
                        }
                    } else {
                        if (it > 0) chain_wait(h);  // the previous tile's dW_0 has left the accumulator
                    }
                    if (h == 0) ok = ok && mbar_wait(&x_full[b], (it >> 1) & 1u, abort_flag, p.status, kStatusCtrlX);
                    if (ok && leader) {
                        const uint32_t acc = tmem_base + kColAcc + (uint32_t)(h * CH);
#pragma unroll
                        for (int k = 0; k < D0 / 16; ++k)
                            umma_f16(acc, desc_k(kW0, 16384u, k), desc_k(xbuf + (uint32_t)h * (uint32_t)(CH * 128), 8192u, k), kIdescFwd0, k > 0);
                        umma_commit(&acc_full[h]);
                        MLPB200_TRACE_AT(tr_on, (tr_step * 2 + h) * 3 + 2);
                    }
                }
#ifdef MLPB200_TRACE
                ++tr_step;
#endif
                // ---- forward, layers 1..3 ----
#pragma unroll
                for (int l = 1; l < NL - 1; ++l) {
                    const uint32_t wpanel = (uint32_t)out_dim(l, NL) * 128u;
                    const uint32_t abuf = kA1 + (uint32_t)(l - 1) * 16384u;
#pragma unroll
                    for (int h = 0; h < NCH; ++h) {
                        chain_wait(h);
                        if (ok && leader) {
                            const uint32_t acc = tmem_base + kColAcc + (uint32_t)(h * CH);
                            const uint32_t half = (uint32_t)h * (uint32_t)(CH * 2);  // the chain's samples inside a feature row
#pragma unroll
                            for (int k = 0; k < H / 16; ++k)
                                umma_f16(acc, desc_k(w_off(l, NL), wpanel, k), desc_mn(abuf + half, 8192u, k), kIdescFwd, k > 0);
                            umma_commit(&acc_full[h]);
                            MLPB200_TRACE_AT(tr_on, (tr_step * 2 + h) * 3 + 2);
                        }
                    }
#ifdef MLPB200_TRACE
                    ++tr_step;
#endif
                }
                // ---- output layer, whole tile: Z_4 [samples x 64] = A_4 [samples x 128] . W_4^T with the samples
                //      on the TMEM lanes.  A_4's rows hold 64 samples; the second half of the 128 lanes reads the
                //      same 64 samples again (panel stride 0), so lanes 64..127 mirror lanes 0..63 and all four
                //      lane quarters can share the output-layer epilogue ----
#pragma unroll
                for (int h = 0; h < NCH; ++h) chain_wait(h);
                if (ok && leader) {
#pragma unroll
                    for (int k = 0; k < H / 16; ++k)
                        umma_f16(tmem_base + kColAcc, desc_mn(kA1 + (uint32_t)(NL - 2) * 16384u, 0u, k), desc_k(kW4, 8192u, k), kIdescOut, k > 0);
                    umma_commit(out_full);
                    MLPB200_TRACE_AT(tr_on, (tr_step * 2 + 0) * 3 + 2);
                }
#ifdef MLPB200_TRACE
                ++tr_step;
#endif
                if constexpr (FWD) {
                    // forward only: the next tile's inputs (the other buffer's last reader was the previous tile's layer 0)
                    if (ok && leader && has_next) {
                        mbar_expect_tx(&x_full[b ^ 1u], 8192);
                        tma_load_2d(smem + kX + (b ^ 1u) * 8192u, &tmap_x, 0, (int32_t)(next_tile * NS), &x_full[b ^ 1u]);
                    }
                    if (has_next) ++loads_issued;
                    continue;
                }
                // ---- backward ----
                MLPB200_TRACE_AT(tr_on, (tr_step * 2 + 0) * 3 + 0);
                ok = ok && mbar_wait(out_free, it & 1u, abort_flag, p.status, kStatusCtrlAcc);  // dZ_4 is in place
                tc_fence_after();
                MLPB200_TRACE_AT(tr_on, (tr_step * 2 + 0) * 3 + 1);
#pragma unroll
                for (int l = NL - 1; l >= 1; --l) {
                    const uint32_t wpanel = (uint32_t)out_dim(l, NL) * 128u;
                    const uint32_t dzbuf = (l == NL - 1) ? kDZ4 : kA1 + (uint32_t)l * 16384u;  // dZ_l lives in A_{l+1}'s buffer
                    const uint32_t abuf = kA1 + (uint32_t)(l - 1) * 16384u;                   // A_l
#pragma unroll
                    for (int h = 0; h < NCH; ++h) {
                        if (l < NL - 1) chain_wait(h);
                        if (ok && leader) {
                            const uint32_t acc = tmem_base + kColAcc + (uint32_t)(h * CH);
                            const uint32_t row = (uint32_t)h * (uint32_t)(CH * 128);  // sample-major tiles: 32 rows of 128 bytes
                            const uint32_t half = (uint32_t)h * (uint32_t)(CH * 2);   // feature-major tiles: 64 bytes inside a row
                            const uint32_t prior = (it > 0 || h > 0) ? 1u : 0u;  // the launch's first product overwrites
                            if (l == NL - 1) {
#pragma unroll
                                for (int k = 0; k < out_dim(l, NL) / 16; ++k)
                                    umma_f16(acc, desc_mn(w_off(l, NL), wpanel, k), desc_k(dzbuf + row, 8192u, k), kIdescDx4, k > 0);
#pragma unroll
                                for (int k = 0; k < CH / 16; ++k)
                                    umma_f16(tmem_base + kColDW4T, desc_k(abuf + half, 0u, k), desc_mn(dzbuf + row, 8192u, k),
                                             kIdescDw64, prior | (uint32_t)(k > 0));
                            } else {
#pragma unroll
                                for (int k = 0; k < out_dim(l, NL) / 16; ++k)
                                    umma_f16(acc, desc_mn(w_off(l, NL), wpanel, k), desc_mn(dzbuf + half, 8192u, k), kIdescDx, k > 0);
#pragma unroll
                                for (int k = 0; k < CH / 16; ++k)
                                    umma_f16(tmem_base + kColDW1 + (uint32_t)(l - 1) * 128u, desc_k(dzbuf + half, 0u, k),
                                             desc_k(abuf + half, 0u, k), kIdescDw, prior | (uint32_t)(k > 0));
                            }
                            umma_commit(&acc_full[h]);
                            MLPB200_TRACE_AT(tr_on, (tr_step * 2 + h) * 3 + 2);
                        }
                    }
#ifdef MLPB200_TRACE
                    ++tr_step;
#endif
                }
                // ---- dW_0 of the whole tile into the 64 accumulator columns (the epilogue adds them to
                //      registers); then the next tile's loads ----
#pragma unroll
                for (int h = 0; h < NCH; ++h) chain_wait(h);
                if (ok) {
                    if (leader) {
#pragma unroll
                        for (int k = 0; k < NS / 16; ++k)
                            umma_f16(tmem_base + kColAcc, desc_k(kA1, 0u, k), desc_mn(xbuf, 8192u, k), kIdescDw64, k > 0);
#pragma unroll
                        for (int h = 0; h < NCH; ++h) umma_commit(&acc_full[h]);
                        MLPB200_TRACE_AT(tr_on, (tr_step * 2 + 0) * 3 + 2);
                        if (has_next) {
                            // Both chains are past every product that read the other X buffer and dZ_4.
                            mbar_expect_tx(&x_full[b ^ 1u], 8192);
                            tma_load_2d(smem + kX + (b ^ 1u) * 8192u, &tmap_x, 0, (int32_t)(next_tile * NS), &x_full[b ^ 1u]);
                            if (!p.t_direct) {
                                mbar_expect_tx(t_full, 8192);
                                tma_load_2d(smem + kDZ4, &tmap_t, 0, (int32_t)(next_tile * NS), t_full);
                            }
                        }
                    }
                    if (has_next) ++loads_issued;
                    __syncwarp();
                }
                // ---- optional: the input gradient dA_0^T [inputs x samples] = W_0^T . dZ_0^T of both chains, once
                //      dW_0 has left the accumulator.  W_0 holds 64 input columns; the instruction's upper 64 lanes
                //      read the rows of the next weight buffer and are never looked at ----
                if (XTRA && p.input_grads) {
#pragma unroll
                    for (int h = 0; h < NCH; ++h) chain_wait(h);
                    if (ok && leader) {
#pragma unroll
                        for (int h = 0; h < NCH; ++h) {
                            const uint32_t half = (uint32_t)h * (uint32_t)(CH * 2);
#pragma unroll
                            for (int k = 0; k < H / 16; ++k)
                                umma_f16(tmem_base + kColAcc + (uint32_t)(h * CH), desc_mn(kW0, 16384u, k), desc_mn(kA1 + half, 8192u, k),
                                         kIdescDx, k > 0);
                        }
#pragma unroll
                        for (int h = 0; h < NCH; ++h) umma_commit(&acc_full[h]);
                    }
                    __syncwarp();
                }
            }
            if (*abort_flag && leader) {
                // Give the copies still in flight a bounded time to land before the CTA exits.
                mbar_drain(&x_full[(loads_issued - 1) & 1u], ((loads_issued - 1) >> 1) & 1u);
                if (!p.t_direct) mbar_drain(t_full, (loads_issued - 1) & 1u);
            }
        }
#ifdef MLPB200_TRACE
    } else if (warp == 1) {
        // Trace builds: the otherwise idle warp watches the accumulator barriers and stamps the moment each
        // chain's products complete, independent of what the epilogue warps are busy with.
        if (blockIdx.x == 0 && p.timing && n_my_tiles > kTraceTile) {
            uint32_t nf[2] = {0, 0};
            bool ok = true;
            for (uint32_t it = 0; it <= kTraceTile && ok; ++it) {
                uint32_t st = 0;
                for (int ph = 0; ph < 10 && ok; ++ph) {
                    if (ph == 4) {
                        ok = mbar_wait(out_full, it & 1u, abort_flag, p.status, kStatusEpiAcc);
                        if (it == kTraceTile && lane == 0) p.timing[200 + st] = (unsigned long long)clock64();
                        st += 2;
                        continue;
                    }
                    for (int h = 0; h < 2 && ok; ++h) {
                        ok = mbar_wait(&acc_full[h], nf[h] & 1u, abort_flag, p.status, kStatusEpiAcc);
                        ++nf[h];
                        if (it == kTraceTile && lane == 0) p.timing[200 + st + h] = (unsigned long long)clock64();
                    }
                    st += 2;
                }
            }
        }
#endif
    } else if (warp >= 2) {
        // =================================== epilogue warps ========================================
        // Hidden layers: a thread owns one feature (TMEM lane f) and, of each chain, the eight sample columns
        // of its column group e, so every warp takes a share of every chain step.  The bias is a
        // per-thread constant and the hidden bias gradients are per-thread sums.
        const int q = warp & 3;                // TMEM lane quarter this warp may read
        const int e = (warp - 2) >> 2;         // column group 0..3
        const int f = q * 32 + lane;           // the feature (TMEM lane) this thread owns
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        // Feature-major tiles ([128 features][64 samples]): this thread's eight samples of chain h are the
        // 16-byte chunk 4h + e of row f, stored at chunk (4h + e) ^ (f & 7).
        const uint32_t frow = (uint32_t)f * 128u;
        auto chunk_of = [&](int h) -> uint32_t { return frow + ((((uint32_t)(h * 4 + e)) ^ (uint32_t)(f & 7)) << 4); };

        uint32_t dreg[NCH][NL - 1][CPT / 2];  // activation derivatives of the four hidden layers, two per register
        float dw0[16];                        // this thread's slice of dW_0 (row f, columns 16e..16e+15), summed over tiles
        float db[NL - 1];                     // hidden bias-gradient partial sums (feature f)
        float db_out = 0.0f;                  // output bias-gradient partial sum (see the output layer)
#pragma unroll
        for (int i = 0; i < 16; ++i) dw0[i] = 0.0f;
#pragma unroll
        for (int l = 0; l < NL - 1; ++l) db[l] = 0.0f;
        float run_max = 0.0f, run_sum = 0.0f;  // per-lane (per sample slot) in the two warps that total the losses
        uint32_t n_full0 = 0, n_full1 = 0;     // phases of acc_full[h] this warp has consumed
        constexpr bool fp32_storage = F32S;  // pre-activations and outputs are not rounded
        bool ok = true;
#ifdef MLPB200_TRACE
        bool tr_on = false;
        uint32_t tr_step = 0;
#endif
        auto wait_acc = [&](int h) {
            uint32_t& n = h == 0 ? n_full0 : n_full1;
            ok = ok && mbar_wait(&acc_full[h], n & 1u, abort_flag, p.status, kStatusEpiAcc);
            ++n;
            MLPB200_TRACE_AT(tr_on, 64u + (uint32_t)h * 64u + tr_step * 4 + 0);
        };
        auto release = [&](uint64_t* bar) {
            tc_fence_before();
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar);
        };

        for (uint32_t it = 0; it < n_my_tiles && ok; ++it) {
            const uint32_t tile = blockIdx.x + it * gridDim.x;
#ifdef MLPB200_TRACE
            tr_on = blockIdx.x == 0 && it == kTraceTile && p.timing && q == 0 && e == 0 && lane == 0;
            tr_step = 0;
#endif
            // ---- forward, hidden layers ----
#pragma unroll
            for (int l = 0; l < NL - 1; ++l) {
                const float bl = s_bias[l * 128 + f];
                const float2 bias2 = make_float2(bl, bl);
#pragma unroll
                for (int h = 0; h < NCH; ++h) {
                    wait_acc(h);
                    if (ok) {
                        tc_fence_after();
                        uint32_t v[CPT];
                        tmem_ld_cols(lane_base + kColAcc + (uint32_t)(h * CH + e * CPT), v);
                        tmem_ld_wait();
                        MLPB200_TRACE_AT(tr_on, 64u + (uint32_t)h * 64u + tr_step * 4 + 1);
                        uint32_t aw[CPT / 2];
#pragma unroll
                        for (int s = 0; s < CPT; s += 2) {
                            // bias, storage rounding of the pre-activation (one paired conversion), activation
                            const float2 zf = __fadd2_rn(make_float2(__uint_as_float(v[s]), __uint_as_float(v[s + 1])), bias2);
                            float2 z = zf;
                            if constexpr (!fp32_storage) {
                                const uint32_t zr = E::pack2(zf.x, zf.y);
                                z = make_float2(E::unpack_lo(zr), E::unpack_hi(zr));
                            }
                            float2 a, d;
                            if constexpr (ACT >= 0) {
                                act_pair2<ACT>(z, p.act_alpha, a, d);
                            } else {
                                act_pair_rt(p.hidden_act, z.x, p.act_alpha, a.x, d.x);
                                act_pair_rt(p.hidden_act, z.y, p.act_alpha, a.y, d.y);
                            }
                            aw[s >> 1] = E::pack2(a.x, a.y);
                            if constexpr (!FWD) dreg[h][l][s >> 1] = E::pack2(d.x, d.y);
                        }
                        *(uint4*)(smem + kA1 + (uint32_t)l * 16384u + chunk_of(h)) = make_uint4(aw[0], aw[1], aw[2], aw[3]);
                        MLPB200_TRACE_AT(tr_on, 64u + (uint32_t)h * 64u + tr_step * 4 + 2);
                        release(&acc_free[h]);
                        MLPB200_TRACE_AT(tr_on, 64u + (uint32_t)h * 64u + tr_step * 4 + 3);
                    }
                }
#ifdef MLPB200_TRACE
                ++tr_step;
#endif
            }
            if (!ok) break;
            // ---- output layer, loss and dZ_4: samples on the lanes.  Lane L of the accumulator holds sample
            //      L % 64 (lanes 64..127 mirror lanes 0..63), so the lane quarters 0, 1 take output features
            //      0..31 and the quarters 2, 3 features 32..63 of the same 64 samples; a thread owns one sample
            //      and eight features: one 16-byte chunk of the target row, replaced in place by dZ_4 ----
            {
                ok = ok && mbar_wait(out_full, it & 1u, abort_flag, p.status, kStatusEpiAcc);
                if (!FWD && !p.t_direct) ok = ok && mbar_wait(t_full, it & 1u, abort_flag, p.status, kStatusEpiTarget);
                if (!ok) break;
                MLPB200_TRACE_AT(tr_on, 64u + tr_step * 4 + 0);
                tc_fence_after();
                const int s = (q & 1) * 32 + lane;             // sample slot inside the tile
                const int fb = (q >> 1) * 32 + e * 8;          // first of this thread's eight output features
                uint32_t v[8];
                tmem_ld_cols(lane_base + kColAcc + (uint32_t)fb, v);
                tmem_ld_wait();
                MLPB200_TRACE_AT(tr_on, 64u + tr_step * 4 + 1);
                const bool valid = tile * NS + (uint32_t)s < p.count;
                if constexpr (FWD) {
                    // the pre-activations of the output layer, rounded to the storage type, as fp32
                    const float4 c0 = *(const float4*)(s_bias + (kMaxLayers - 1) * 128 + fb);
                    const float4 c1 = *(const float4*)(s_bias + (kMaxLayers - 1) * 128 + fb + 4);
                    const float bb[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                    const int od = p.dims[NL];
                    if (valid) {
                        float* dst = p.outputs + ((size_t)tile * NS + (size_t)s) * (size_t)od + fb;
#pragma unroll
                        for (int j = 0; j < 8; j += 2) {
                            const float r0 = __uint_as_float(v[j]) + bb[j], r1 = __uint_as_float(v[j + 1]) + bb[j + 1];
                            const uint32_t op = E::pack2(r0, r1);
                            if (fb + j < od) dst[j] = fp32_storage ? r0 : E::unpack_lo(op);
                            if (fb + j + 1 < od) dst[j + 1] = fp32_storage ? r1 : E::unpack_hi(op);
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(out_free);
                    continue;
                }
                uint4* slot = (uint4*)(smem + kDZ4 + (uint32_t)s * 128u + ((((uint32_t)(fb >> 3)) ^ (uint32_t)(s & 7)) << 4));
                float tf[8];
                if (!p.t_direct) {
                    const uint4 tq = *slot;
                    const uint32_t tw[4] = {tq.x, tq.y, tq.z, tq.w};
#pragma unroll
                    for (int j = 0; j < 8; j += 2) { tf[j] = E::unpack_lo(tw[j >> 1]); tf[j + 1] = E::unpack_hi(tw[j >> 1]); }
                } else {
                    // targets of any width or number format: this sample's eight features straight from global memory
                    const int od = p.dims[NL];
                    const size_t row = ((size_t)tile * NS + (size_t)s) * (size_t)od;
#pragma unroll
                    for (int j = 0; j < 8; ++j) tf[j] = (valid && fb + j < od) ? load_as_f32(p.target_dtype, p.targets, (int64_t)(row + fb + j)) : 0.0f;
                }
                const float4 b0 = *(const float4*)(s_bias + (kMaxLayers - 1) * 128 + fb);
                const float4 b1 = *(const float4*)(s_bias + (kMaxLayers - 1) * 128 + fb + 4);
                const float bo[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                const float two_scale = 2.0f * p.loss_scale;
                float dzf[8];
                uint32_t zw[4];
                float loss = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float r0 = __uint_as_float(v[j]) + bo[j], r1 = __uint_as_float(v[j + 1]) + bo[j + 1];
                    const uint32_t op = E::pack2(r0, r1);  // storage rounding
                    const float d0 = (fp32_storage ? r0 : E::unpack_lo(op)) - tf[j];
                    const float d1 = (fp32_storage ? r1 : E::unpack_hi(op)) - tf[j + 1];
                    const uint32_t zp = valid ? E::pack2(two_scale * d0, two_scale * d1) : 0u;
                    zw[j >> 1] = zp;
                    dzf[j] = E::unpack_lo(zp);
                    dzf[j + 1] = E::unpack_hi(zp);
                    if (valid) {
                        loss = fmaf(d0 * p.loss_scale, d0, loss);
                        loss = fmaf(d1 * p.loss_scale, d1, loss);
                    }
                }
                *slot = make_uint4(zw[0], zw[1], zw[2], zw[3]);
                s_loss_part[((q >> 1) * 4 + e) * 64 + s] = loss;
                MLPB200_TRACE_AT(tr_on, 64u + tr_step * 4 + 2);
                release(out_free);  // dZ_4 and this warp's loss terms are in place
                MLPB200_TRACE_AT(tr_on, 64u + tr_step * 4 + 3);
                // Output bias gradient: sum each of the eight features over the warp's 32 samples.  Every
                // exchange round halves the number of features a lane carries; after three rounds and two
                // full rounds, lane carries the total of feature fb + 4 * bit4 + 2 * bit3 + bit2 of its index.
                {
                    const bool u16 = (lane & 16) != 0, u8 = (lane & 8) != 0, u4 = (lane & 4) != 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float keep = u16 ? dzf[i + 4] : dzf[i];
                        const float send = u16 ? dzf[i] : dzf[i + 4];
                        dzf[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const float keep = u8 ? dzf[i + 2] : dzf[i];
                        const float send = u8 ? dzf[i] : dzf[i + 2];
                        dzf[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
                    }
                    {
                        const float keep = u4 ? dzf[1] : dzf[0];
                        const float send = u4 ? dzf[0] : dzf[1];
                        dzf[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
                    }
                    dzf[0] += __shfl_xor_sync(0xffffffffu, dzf[0], 2);
                    dzf[0] += __shfl_xor_sync(0xffffffffu, dzf[0], 1);
                    db_out += dzf[0];
                }
                if (e == 0 && q < 2) {
                    // This warp totals the per-sample losses of its 32 samples once every warp has written its terms.
                    ok = ok && mbar_wait(out_free, it & 1u, abort_flag, p.status, kStatusEpiLoss);
                    if (!ok) break;
                    float tot = 0.0f;
#pragma unroll
                    for (int g = 0; g < 8; ++g) tot += s_loss_part[g * 64 + s];
                    run_max = fmaxf(run_max, tot);
                    run_sum += tot;
                }
#ifdef MLPB200_TRACE
                ++tr_step;
#endif
            }
            // ---- backward: dA_l arrives in the accumulator, dZ_{l-1} replaces A_l in shared memory ----
#pragma unroll
            for (int l = NL - 1; l >= 1; --l) {
#pragma unroll
                for (int h = 0; h < NCH; ++h) {
                    wait_acc(h);
                    if (ok) {
                        tc_fence_after();
                        uint32_t v[CPT];
                        tmem_ld_cols(lane_base + kColAcc + (uint32_t)(h * CH + e * CPT), v);
                        tmem_ld_wait();
                        MLPB200_TRACE_AT(tr_on, 64u + (uint32_t)h * 64u + tr_step * 4 + 1);
                        float2 dbp = make_float2(0.0f, 0.0f);
                        uint32_t zw[CPT / 2];
#pragma unroll
                        for (int s = 0; s < CPT; s += 2) {
                            const uint32_t dd = dreg[h][l - 1][s >> 1];
                            const float2 g = __fmul2_rn(make_float2(__uint_as_float(v[s]), __uint_as_float(v[s + 1])),
                                                        make_float2(E::unpack_lo(dd), E::unpack_hi(dd)));
                            const uint32_t zp = E::pack2(g.x, g.y);
                            zw[s >> 1] = zp;
                            dbp = __fadd2_rn(dbp, make_float2(E::unpack_lo(zp), E::unpack_hi(zp)));
                        }
                        *(uint4*)(smem + kA1 + (uint32_t)(l - 1) * 16384u + chunk_of(h)) = make_uint4(zw[0], zw[1], zw[2], zw[3]);
                        db[l - 1] += dbp.x + dbp.y;
                        MLPB200_TRACE_AT(tr_on, 64u + (uint32_t)h * 64u + tr_step * 4 + 2);
                        release(&acc_free[h]);
                        MLPB200_TRACE_AT(tr_on, 64u + (uint32_t)h * 64u + tr_step * 4 + 3);
                    }
                }
#ifdef MLPB200_TRACE
                ++tr_step;
#endif
            }
            if (!ok) break;
            // ---- dW_0 of this tile: add the accumulator to the register slice ----
            {
                wait_acc(0);
                wait_acc(1);
                if (!ok) break;
                tc_fence_after();
                uint32_t v[16];
                tmem_ld_cols(lane_base + kColAcc + (uint32_t)(e * 16), v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) dw0[i] += __uint_as_float(v[i]);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&acc_free[0]);
                    mbar_arrive(&acc_free[1]);
                }
                MLPB200_TRACE_AT(tr_on, 64u + tr_step * 4 + 3);
            }
            // ---- optional: the input gradients of this tile, input feature on the lane (quarters 0 and 1), sample
            //      on the column; a warp writes 32 consecutive features of one sample per store ----
            if (XTRA && p.input_grads) {
                wait_acc(0);
                wait_acc(1);
                if (!ok) break;
                tc_fence_after();
                if (q < 2) {
                    uint32_t v[16];
                    tmem_ld_cols(lane_base + kColAcc + (uint32_t)(e * 16), v);
                    tmem_ld_wait();
                    const int in0 = p.dims[0];
                    if (f < in0) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const size_t sample = (size_t)tile * NS + (size_t)(e * 16 + i);
                            const float g = __uint_as_float(v[i]);
                            if (sample < p.count) p.input_grads[sample * (size_t)in0 + f] = fp32_storage ? g : E::unpack_lo(E::pack2(g, 0.0f));
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&acc_free[0]);
                    mbar_arrive(&acc_free[1]);
                }
            }
        }

        // ---- one add per parameter per CTA ----
        if (!FWD && ok && !*abort_flag && n_my_tiles > 0) {
            tc_fence_after();
            // Only real rows and columns leave; the gradients are row-major [out][in] with the network's own widths.
#pragma unroll
            for (int l = 1; l <= NL - 2; ++l) {
                const int in = p.dims[l], out = p.dims[l + 1];
                float* dW = (float*)p.net[l].weightsGrad + (size_t)f * in;
                const int col = e * 32;
                uint32_t v[32];
                tmem_ld_cols(lane_base + kColDW1 + (uint32_t)(l - 1) * 128u + (uint32_t)col, v);
                tmem_ld_wait();
                if (f < out) {
                    if (XTRA && p.param_layout != MLP_PARAMS_ROW_MAJOR) {
                        // tiled parameters: the gradient of weight (f, i) goes where the weight itself lies
                        float* gW = (float*)p.net[l].weightsGrad;
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col + i < in) atomicAdd(gW + weight_index(p.param_layout, in, out, f, col + i), __uint_as_float(v[i]));
                    } else if ((in & 3) == 0) {
                        // four parameters per reduction (16-byte aligned: rows are multiples of 16 bytes)
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            if (col + i < in)
                                atomicAdd((float4*)(dW + col + i), make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                                                                               __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col + i < in) atomicAdd(dW + col + i, __uint_as_float(v[i]));
                    }
                }
            }
            {
                // dW of the output layer, transposed: lane = input feature, column = output feature.
                const int in = p.dims[NL - 1], out = p.dims[NL];
                float* dW = (float*)p.net[NL - 1].weightsGrad;
                uint32_t v[16];
                tmem_ld_cols(lane_base + kColDW4T + (uint32_t)(e * 16), v);
                tmem_ld_wait();
                if (f < in) {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (e * 16 + i < out) atomicAdd(dW + (XTRA ? weight_index(p.param_layout, in, out, e * 16 + i, f) : (int64_t)(e * 16 + i) * in + f), __uint_as_float(v[i]));
                }
            }
            {
                const int in = p.dims[0], out = p.dims[1];
                float* dW = (float*)p.net[0].weightsGrad + (size_t)f * in + e * 16;
                if (f < out) {
                    if (XTRA && p.param_layout != MLP_PARAMS_ROW_MAJOR) {
                        float* gW = (float*)p.net[0].weightsGrad;
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (e * 16 + i < in) atomicAdd(gW + weight_index(p.param_layout, in, out, f, e * 16 + i), dw0[i]);
                    } else if ((in & 3) == 0) {
#pragma unroll
                        for (int i = 0; i < 16; i += 4)
                            if (e * 16 + i < in) atomicAdd((float4*)(dW + i), make_float4(dw0[i], dw0[i + 1], dw0[i + 2], dw0[i + 3]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (e * 16 + i < in) atomicAdd(dW + i, dw0[i]);
                    }
                }
            }
#pragma unroll
            for (int l = 0; l < NL - 1; ++l)
                if (f < p.dims[l + 1]) atomicAdd((float*)p.net[l].biasesGrad + f, db[l]);
            if ((lane & 3) == 0) {
                const int j = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
                const int feat = (q >> 1) * 32 + e * 8 + j;
                if (feat < p.dims[NL]) atomicAdd((float*)p.net[NL - 1].biasesGrad + feat, db_out);
            }
            if (e == 0 && q < 2) {
                float mx = run_max, tot = run_sum;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    tot += __shfl_xor_sync(0xffffffffu, tot, o);
                }
                if (lane == 0) {
                    atomicMax(p.loss_words, __float_as_uint(mx));
                    atomicAdd((float*)(p.loss_words + 1), tot);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, wide::kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------------
// Host side.  This file is compiled three times (slang_b200/build.py): MLPB200_WIDE_PART 0 holds the workspace,
// the tensor-map helper and the plain training builds of the kernel, part 1 the forward-only builds, part 2
// the training builds with input gradients and tiled-layout gradients.
// ------------------------------------------------------------------------------------------------
#ifndef MLPB200_WIDE_PART
#error "compile with -DMLPB200_WIDE_PART=0, 1 or 2"
#endif
// fp32 input rows -> the operand type, for networks whose inputs arrive as fp32 (an encoder in front of the
// network writes fp32 features): the wide kernel takes its input tile by TMA in the operand type, so the rows
// are rounded once by this launch, exactly as the epilogue-built input rows of the padded kernel are.
template <int FMT>
__global__ void convert_input_rows_kernel(const float4* __restrict__ src, uint2* __restrict__ dst, size_t n4)
{
    using E = Elem<FMT>;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = src[i];
        dst[i] = make_uint2(E::pack2(v.x, v.y), E::pack2(v.z, v.w));
    }
}

// The 16-bit copy of `count` fp32 rows of `width` (a multiple of 8) values; the scratch buffer grows on demand.
static cudaError_t converted_input_rows(cudaStream_t st, TcWorkspace* ws, int op, uint64_t inputs, uint32_t count, int width,
                                        uint64_t* out_address, int* launches)
{
    const size_t n = (size_t)count * (size_t)width;
    if (n * 2 > ws->input_rows_bytes) {
        cudaError_t e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) return e;
        if (ws->input_rows) cudaFree(ws->input_rows);
        ws->input_rows = nullptr;
        ws->input_rows_bytes = 0;
        e = cudaMalloc(&ws->input_rows, n * 2);
        if (e != cudaSuccess) return e;
        ws->input_rows_bytes = n * 2;
    }
    if (inputs & 15u) return cudaErrorMisalignedAddress;
    const size_t n4 = n / 4;
    const unsigned grid = (unsigned)((n4 + 255) / 256 < (size_t)(ws->sm_count * 16) ? (n4 + 255) / 256 : (size_t)(ws->sm_count * 16));
    if (op == MLP_BF16) convert_input_rows_kernel<MLP_BF16><<<grid, 256, 0, st>>>((const float4*)inputs, (uint2*)ws->input_rows, n4);
    else convert_input_rows_kernel<MLP_F16><<<grid, 256, 0, st>>>((const float4*)inputs, (uint2*)ws->input_rows, n4);
    *out_address = (uint64_t)ws->input_rows;
    *launches += 1;
    return cudaGetLastError();
}

static bool wide_supported(const MlpConfig& c)
{
    // Two to five layers; inputs and outputs up to 64 wide, hidden layers up to 128; at least one width
    // above 64 (narrower networks run the padded 64-wide kernel); 16-bit storage with inputs in the same
    // format and rows that start on 16-byte boundaries (the input tile arrives by TMA); identity output.
    const int nl = c.n_layers;
    if (nl < 2 || nl > wide::kMaxLayers) return false;
    const int op = c.operand_dtype ? c.operand_dtype : c.dtype;  // fp32 storage runs here with 16-bit operands
    if (op != MLP_BF16 && op != MLP_F16) return false;
    if (c.input_dtype != op && c.input_dtype != MLP_F32) return false;  // fp32 rows are converted by a launch in front
    if (c.output_act != MLP_ACT_IDENTITY || c.encoding != MLP_ENC_NONE) return false;
    if (c.dims[0] > wide::D0 || (c.dims[0] & 7) != 0 || c.dims[nl] > wide::DOUT) return false;
    bool any_wide = false;
    for (int l = 1; l < nl; ++l) {
        if (c.dims[l] > wide::H) return false;
        any_wide = any_wide || c.dims[l] > 64;
    }
    return any_wide;
}


#if MLPB200_WIDE_PART == 0

bool tc_train_supported(const MlpConfig& c) { return wide_supported(c) || tc_train_narrow_supported(c); }

TcWorkspace* tc_workspace_create(int ordinal, std::string* err)
{
    TcWorkspace* ws = new TcWorkspace();
    ws->ordinal = ordinal;
    cudaError_t e = cudaDeviceGetAttribute(&ws->sm_count, cudaDevAttrMultiProcessorCount, ordinal);
    if (e == cudaSuccess) e = cudaMalloc((void**)&ws->status, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ws->status, 0, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMallocHost((void**)&ws->status_host, sizeof(uint32_t));
#ifdef MLPB200_TRACE
    if (e == cudaSuccess) e = cudaMalloc((void**)&ws->timing, 256 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(ws->timing, 0, 256 * sizeof(unsigned long long));
#endif
    if (e == cudaSuccess) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e == cudaSuccess && (qres != cudaDriverEntryPointSuccess || !fn)) e = cudaErrorNotSupported;
        ws->encode = (EncodeTiledFn)fn;
    }
    if (e != cudaSuccess) {
        if (err) *err = cudaGetErrorString(e);
        tc_workspace_destroy(ws);
        return nullptr;
    }
    return ws;
}

void tc_workspace_destroy(TcWorkspace* ws)
{
    if (!ws) return;
    if (ws->status) cudaFree(ws->status);
    if (ws->status_host) cudaFreeHost(ws->status_host);
    if (ws->timing) cudaFree(ws->timing);
    if (ws->input_rows) cudaFree(ws->input_rows);
    delete ws;
}

#ifdef MLPB200_TRACE
cudaError_t tc_read_timing(cudaStream_t st, TcWorkspace* ws, unsigned long long* out256)
{
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return e;
    return cudaMemcpy(out256, ws->timing, 256 * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
}
#endif

cudaError_t tc_read_status(cudaStream_t st, TcWorkspace* ws, uint32_t* status)
{
    cudaError_t e = cudaMemcpyAsync(ws->status_host, ws->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return e;
    *status = *ws->status_host;
    if (*status) e = cudaMemsetAsync(ws->status, 0, sizeof(uint32_t), st);
    return e;
}

bool make_tile_map(TcWorkspace* ws, CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, uint64_t base, uint64_t rows,
                   uint32_t cols, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle, std::string* err)
{
    if (base & 15u) { if (err) *err = "inputs, targets and outputs must be 16-byte aligned for the TMA path"; return false; }
    const cuuint64_t gdim[2] = {cols, rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)cols * elem_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = ws->encode(map, type, 2, (void*)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { if (err) *err = "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r); return false; }
    return true;
}

#endif  // part 0

template <int FMT, int ACT, int NL, bool FWD, bool F32S = false, bool XTRA = false>
static cudaError_t launch_wide(cudaStream_t st, TcWorkspace* ws, const CUtensorMap& mx, const CUtensorMap& mt,
                               const WideTrainParams& p)
{
    auto kern = learn_gradient_wide_kernel<FMT, ACT, NL, FWD, F32S, XTRA>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wide::kSmemBytes);
    if (e != cudaSuccess) return e;
    const uint32_t grid = p.n_tiles < (uint32_t)ws->sm_count ? p.n_tiles : (uint32_t)ws->sm_count;
    kern<<<grid, wide::kThreads, wide::kSmemBytes, st>>>(mx, mt, p);
    return cudaGetLastError();
}

// The builds of the kernel: GELU (tanh form) and ReLU as compile-time activations for every layer count,
// leaky ReLU for five layers, and every layer count with the activation chosen at run time (slower: every
// element goes through a switch and the library's scalar math).
template <int FMT, bool FWD, bool XTRA = false>
static cudaError_t launch_wide_fmt(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const CUtensorMap& mx,
                                   const CUtensorMap& mt, const WideTrainParams& p)
{
    const int act = c.hidden_act;
    if (c.dtype == MLP_F32) {   // fp32 storage, 16-bit operands
        switch (c.n_layers) {
        case 5: return launch_wide<FMT, -1, 5, FWD, true, XTRA>(st, ws, mx, mt, p);
        case 4: return launch_wide<FMT, -1, 4, FWD, true, XTRA>(st, ws, mx, mt, p);
        case 3: return launch_wide<FMT, -1, 3, FWD, true, XTRA>(st, ws, mx, mt, p);
        case 2: return launch_wide<FMT, -1, 2, FWD, true, XTRA>(st, ws, mx, mt, p);
        }
        return cudaErrorInvalidValue;
    }
    switch (c.n_layers) {
    case 5:
        if (act == MLP_ACT_GELU_TANH) return launch_wide<FMT, MLP_ACT_GELU_TANH, 5, FWD, false, XTRA>(st, ws, mx, mt, p);
        if (act == MLP_ACT_RELU) return launch_wide<FMT, MLP_ACT_RELU, 5, FWD, false, XTRA>(st, ws, mx, mt, p);
        if (act == MLP_ACT_LEAKY_RELU) return launch_wide<FMT, MLP_ACT_LEAKY_RELU, 5, FWD, false, XTRA>(st, ws, mx, mt, p);
        return launch_wide<FMT, -1, 5, FWD, false, XTRA>(st, ws, mx, mt, p);
    case 4:
        if (act == MLP_ACT_GELU_TANH) return launch_wide<FMT, MLP_ACT_GELU_TANH, 4, FWD, false, XTRA>(st, ws, mx, mt, p);
        if (act == MLP_ACT_RELU) return launch_wide<FMT, MLP_ACT_RELU, 4, FWD, false, XTRA>(st, ws, mx, mt, p);
        return launch_wide<FMT, -1, 4, FWD, false, XTRA>(st, ws, mx, mt, p);
    case 3:
        if (act == MLP_ACT_GELU_TANH) return launch_wide<FMT, MLP_ACT_GELU_TANH, 3, FWD, false, XTRA>(st, ws, mx, mt, p);
        if (act == MLP_ACT_RELU) return launch_wide<FMT, MLP_ACT_RELU, 3, FWD, false, XTRA>(st, ws, mx, mt, p);
        return launch_wide<FMT, -1, 3, FWD, false, XTRA>(st, ws, mx, mt, p);
    case 2:
        if (act == MLP_ACT_GELU_TANH) return launch_wide<FMT, MLP_ACT_GELU_TANH, 2, FWD, false, XTRA>(st, ws, mx, mt, p);
        if (act == MLP_ACT_RELU) return launch_wide<FMT, MLP_ACT_RELU, 2, FWD, false, XTRA>(st, ws, mx, mt, p);
        return launch_wide<FMT, -1, 2, FWD, false, XTRA>(st, ws, mx, mt, p);
    }
    return cudaErrorInvalidValue;
}

// Part 2: the training builds with the extras, behind one function for part 0 to call.
cudaError_t launch_wide_train_extras(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, int op, const CUtensorMap& mx,
                                     const CUtensorMap& mt, const WideTrainParams& p);
#if MLPB200_WIDE_PART == 2
cudaError_t launch_wide_train_extras(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, int op, const CUtensorMap& mx,
                                     const CUtensorMap& mt, const WideTrainParams& p)
{
    return op == MLP_BF16 ? launch_wide_fmt<MLP_BF16, false, true>(st, ws, c, mx, mt, p)
                          : launch_wide_fmt<MLP_F16, false, true>(st, ws, c, mx, mt, p);
}
#endif

#if MLPB200_WIDE_PART == 0
cudaError_t launch_learn_gradient_tc(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const MlpLearnGradParamsEx& a,
                                     int* launches, std::string* err, float* input_grads)
{
    if (!wide_supported(c)) return launch_learn_gradient_narrow(st, ws, c, a, launches, err, input_grads);
    if (a.count == 0) return cudaSuccess;
    const int nl = c.n_layers;
    const int d0 = c.dims[0], dout = c.dims[nl];
    CUtensorMap mx, mt;
    const int op = c.operand_dtype ? c.operand_dtype : c.dtype;
    const CUtensorMapDataType dt = op == MLP_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    uint64_t inputs = a.inputs;
    if (c.input_dtype != op) {
        const cudaError_t ce = converted_input_rows(st, ws, op, a.inputs, a.count, d0, &inputs, launches);
        if (ce != cudaSuccess) { if (err) *err = "converting the fp32 input rows failed"; return ce; }
    }
    // Boxes of 64 rows x 64 columns over [count][width]: columns past the real width arrive as zeros.
    if (!make_tile_map(ws, &mx, dt, 2, inputs, a.count, (uint32_t)d0, 64, wide::NS, CU_TENSOR_MAP_SWIZZLE_128B, err)) return cudaErrorInvalidValue;
    // Targets come by TMA when their rows are 16-byte multiples in the storage format, else the epilogue reads them.
    const bool t_direct = c.target_dtype != op || (dout & 7) != 0 || (a.targets & 15u) != 0;
    if (t_direct) mt = mx;
    else if (!make_tile_map(ws, &mt, dt, 2, a.targets, a.count, (uint32_t)dout, 64, wide::NS, CU_TENSOR_MAP_SWIZZLE_128B, err)) return cudaErrorInvalidValue;
    WideTrainParams p;
    for (int l = 0; l <= wide::kMaxLayers; ++l) p.dims[l] = l <= nl ? c.dims[l] : 0;
    p.hidden_act = c.hidden_act;
    p.param_layout = c.param_layout;
    p.storage_dtype = c.dtype;
    p.t_direct = t_direct ? 1 : 0;
    p.target_dtype = c.target_dtype;
    p.targets = (const void*)a.targets;
    p.net = (const MlpLayerPointers*)a.networkBuffer;
    p.loss_words = (uint32_t*)a.lossBuffer;
    p.status = ws->status;
    p.count = a.count;
    p.n_tiles = (a.count + wide::NS - 1) / wide::NS;
    p.loss_scale = c.loss == MLP_LOSS_MSE_MEAN ? 1.0f / (float)dout : 1.0f;
    p.act_alpha = c.act_alpha;
    p.timing = ws->timing;
    p.outputs = nullptr;
    p.input_grads = input_grads;
    const bool extras = input_grads != nullptr || c.param_layout != MLP_PARAMS_ROW_MAJOR;
    const cudaError_t e = extras ? launch_wide_train_extras(st, ws, c, op, mx, mt, p)
                          : op == MLP_BF16 ? launch_wide_fmt<MLP_BF16, false>(st, ws, c, mx, mt, p)
                                           : launch_wide_fmt<MLP_F16, false>(st, ws, c, mx, mt, p);
    *launches += 1;
    return e;
}
#elif MLPB200_WIDE_PART == 1  // the forward entry point of the same shapes

bool tc_forward_wide_supported(const MlpConfig& c) { return wide_supported(c); }

cudaError_t launch_forward_wide(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const MlpForwardParams& a,
                                int* launches, std::string* err)
{
    if (!wide_supported(c)) { if (err) *err = "shape not built for the wide tensor-core path"; return cudaErrorInvalidValue; }
    if (a.count == 0) return cudaSuccess;
    const int nl = c.n_layers;
    CUtensorMap mx;
    const int op = c.operand_dtype ? c.operand_dtype : c.dtype;
    const CUtensorMapDataType dt = op == MLP_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    uint64_t inputs = a.inputs;
    if (c.input_dtype != op) {
        const cudaError_t ce = converted_input_rows(st, ws, op, a.inputs, a.count, c.dims[0], &inputs, launches);
        if (ce != cudaSuccess) { if (err) *err = "converting the fp32 input rows failed"; return ce; }
    }
    if (!make_tile_map(ws, &mx, dt, 2, inputs, a.count, (uint32_t)c.dims[0], 64, wide::NS, CU_TENSOR_MAP_SWIZZLE_128B, err)) return cudaErrorInvalidValue;
    WideTrainParams p;
    for (int l = 0; l <= wide::kMaxLayers; ++l) p.dims[l] = l <= nl ? c.dims[l] : 0;
    p.hidden_act = c.hidden_act;
    p.param_layout = c.param_layout;
    p.storage_dtype = c.dtype;
    p.t_direct = 1;
    p.target_dtype = c.target_dtype;
    p.targets = nullptr;
    p.outputs = (float*)a.outputs;
    p.net = (const MlpLayerPointers*)a.networkBuffer;
    p.loss_words = nullptr;
    p.status = ws->status;
    p.count = a.count;
    p.n_tiles = (a.count + wide::NS - 1) / wide::NS;
    p.loss_scale = 1.0f;
    p.act_alpha = c.act_alpha;
    p.timing = nullptr;
    p.input_grads = nullptr;
    const cudaError_t e = op == MLP_BF16 ? launch_wide_fmt<MLP_BF16, true>(st, ws, c, mx, mx, p)
                                              : launch_wide_fmt<MLP_F16, true>(st, ws, c, mx, mx, p);
    *launches += 1;
    return e;
}
#endif

}  // namespace mlpb200
