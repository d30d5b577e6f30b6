// Tensor-core (tcgen05 / TMEM / TMA) kernels for sm_100a.
//
// learnGradient for the wide network 64 -> 128 -> 128 -> 128 -> 128 -> 64 (16-bit storage, fp32
// accumulate): one persistent CTA per SM walks 64-sample tiles.  All five weight matrices stay in
// shared memory for the whole launch, every layer product of the forward and backward pass is a
// tcgen05.mma with the accumulator in tensor memory, the weight-gradient products accumulate in
// tensor memory across all of the CTA's tiles, and each parameter receives one atomic add per CTA at
// the end.  Activations never leave the SM.
//
// Orientation: features run along the 128 TMEM lanes (the MMA's M), samples along the columns (N = 64):
//   forward   Z_l^T [out x 64]  = W_l [out x in]   . A_l^T          A: W_l, K-major      B: A_l,  K-major
//   input     dA_l^T [in x 64]  = W_l^T [in x out] . dZ_l^T         A: W_l, MN-major     B: dZ_l, K-major
//   weights   dW_l [out x in]  += dZ_l^T [out x 64] . A_l [64 x in]  A: dZ_l, MN-major    B: A_l,  MN-major
// so a single copy of W_l (row-major rows of 128 bytes, 128-byte swizzle) serves both directions and
// each activation / gradient tile [64 samples][features] serves as a K-major and an MN-major operand.
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
#include "tc_ptx.cuh"

namespace mlpb200 {

using namespace ptx;

// Status-word codes (which wait gave up).
enum : uint32_t {
    kStatusCtrlAcc = 1u, kStatusCtrlX = 2u, kStatusEpiAcc = 4u, kStatusEpiTarget = 8u, kStatusEpiLoss = 16u,
};

namespace wide {
constexpr int NS = 64;            // samples per tile (MMA N of the forward / input-gradient products)
constexpr int D0 = 64, H = 128, DOUT = 64, NL = 5;
constexpr int kThreads = 320;     // warp 0: TMA + MMA issue, warp 1: TMEM owner, warps 2-9: epilogue
constexpr int kEpiThreads = 256;

// Shared-memory map (bytes from a 1024-aligned base).  Operand buffers are panels of
// [rows][128 bytes] with the 128-byte swizzle; a panel holds 64 16-bit features of every row.
constexpr uint32_t kW0 = 0;                  // 128 rows x 1 panel
constexpr uint32_t kW1 = 16384;              // 128 rows x 2 panels (panel stride 16384)
constexpr uint32_t kW2 = kW1 + 32768;
constexpr uint32_t kW3 = kW2 + 32768;
constexpr uint32_t kW4 = kW3 + 32768;        // 64 rows x 2 panels (panel stride 8192)
constexpr uint32_t kX = kW4 + 16384;         // 2 buffers x [64 rows x 1 panel]
constexpr uint32_t kA1 = kX + 2 * 8192;      // A_1..A_4: [64 rows x 2 panels] each (panel stride 8192)
constexpr uint32_t kDZ4 = kA1 + 4 * 16384;   // [64 rows x 1 panel]: targets land here, dZ_4 replaces them
constexpr uint32_t kBias = kDZ4 + 8192;      // fp32 [5][128]
constexpr uint32_t kLossPart = kBias + 5 * 128 * 4;  // fp32 [2][64]
constexpr uint32_t kBars = kLossPart + 2 * 64 * 4;   // mbarriers: x_full[2], t_full, acc_full, acc_free, loss_bar
constexpr uint32_t kTmemPtr = kBars + 8 * 8;
constexpr uint32_t kAbort = kTmemPtr + 4;
constexpr uint32_t kSmemBytes = kAbort + 4 + 1024;   // + slack for aligning the base

// Tensor-memory columns.
constexpr uint32_t kColDW1 = 0, kColDW4T = 384, kColAcc = 448, kTmemCols = 512;

__host__ __device__ constexpr uint32_t w_off(int l) { return l == 0 ? kW0 : l == 1 ? kW1 : l == 2 ? kW2 : l == 3 ? kW3 : kW4; }
__host__ __device__ constexpr int in_dim(int l) { return l == 0 ? D0 : H; }
__host__ __device__ constexpr int out_dim(int l) { return l == NL - 1 ? DOUT : H; }
}  // namespace wide

template <int FMT> struct Elem;
template <> struct Elem<MLP_BF16> {
    static constexpr uint32_t kUmmaFmt = 1;
    __device__ static __forceinline__ uint16_t pack(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }
    __device__ static __forceinline__ float unpack(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
    __device__ static __forceinline__ float round(float v) { return unpack(pack(v)); }
};
template <> struct Elem<MLP_F16> {
    static constexpr uint32_t kUmmaFmt = 0;
    __device__ static __forceinline__ uint16_t pack(float v) { return __half_as_ushort(__float2half_rn(v)); }
    __device__ static __forceinline__ float unpack(uint16_t b) { return __half2float(__ushort_as_half(b)); }
    __device__ static __forceinline__ float round(float v) { return unpack(pack(v)); }
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

struct WideTrainParams {
    const MlpLayerPointers* net;
    uint32_t* loss_words;
    uint32_t* status;
    uint32_t count;
    uint32_t n_tiles;
    float loss_scale;  // 1 / outputs for the mean-squared error, 1 for the sum of squares
    float act_alpha;
};

template <int FMT, int ACT>
__global__ void __launch_bounds__(wide::kThreads, 1)
learn_gradient_wide_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_t,
                           const WideTrainParams p)
{
    using namespace wide;
    using E = Elem<FMT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    uint64_t* bars = (uint64_t*)(smem + kBars);
    uint64_t* x_full = bars;  // [2]
    uint64_t* t_full = bars + 2;
    uint64_t* acc_full = bars + 3;
    uint64_t* acc_free = bars + 4;
    uint64_t* loss_bar = bars + 5;
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
        mbar_init(acc_full, 1);
        mbar_init(acc_free, kEpiThreads / 32);
        mbar_init(loss_bar, 4);
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
        const int in = in_dim(l), out = out_dim(l);
        const uint4* src = (const uint4*)p.net[l].weights;  // 16-byte chunks: 8 elements
        const int chunks_per_row = in / 8;
        const uint32_t panel_stride = (uint32_t)out * 128u;
        for (int idx = threadIdx.x; idx < out * chunks_per_row; idx += kThreads) {
            const int o = idx / chunks_per_row, c = idx % chunks_per_row;
            const uint4 v = src[idx];
            const uint32_t off = w_off(l) + (uint32_t)(c >> 3) * panel_stride + (uint32_t)o * 128u + (uint32_t)(((c & 7) ^ (o & 7)) << 4);
            *(uint4*)(smem + off) = v;
        }
        for (int j = threadIdx.x; j < 128; j += kThreads)
            s_bias[l * 128 + j] = j < out ? load_as_f32(FMT, (const void*)p.net[l].biases, j) : 0.0f;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    if (warp == 0) {
        // =================================== control thread ========================================
        if (lane == 0 && n_my_tiles > 0) {
            constexpr uint32_t F = E::kUmmaFmt;
            constexpr uint32_t kIdescFwd = umma_idesc(F, 0, 0, 128, NS);    // W (K) x act (K)
            constexpr uint32_t kIdescDx = umma_idesc(F, 1, 0, 128, NS);     // W^T (MN) x dZ (K)
            constexpr uint32_t kIdescDw = umma_idesc(F, 1, 1, 128, 128);    // dZ^T (MN) x act (MN)
            constexpr uint32_t kIdescDw64 = umma_idesc(F, 1, 1, 128, 64);   // N = 64 variants (dW_4^T, dW_0)
            const uint32_t acc = tmem_base + kColAcc;
            uint32_t step = 0;
            bool ok = true;
            auto acc_wait = [&]() {
                if (step > 0) ok = ok && mbar_wait(acc_free, (step - 1) & 1u, abort_flag, p.status, kStatusCtrlAcc);
                tc_fence_after();
            };
            // K-major operand: rows of 128 bytes, 8-row groups 1024 bytes apart; a K step of 16
            // elements is 32 bytes inside the swizzled row; 64-element panels are `panel` bytes apart.
            auto desc_k = [&](uint32_t buf, uint32_t panel, int k) {
                return smem_desc_sw128(sbase + buf + (uint32_t)(k >> 2) * panel + (uint32_t)(k & 3) * 32u, 16u, 1024u);
            };
            // MN-major operand: a K step of 16 rows is 2048 bytes; 64-element panels are `panel` bytes apart.
            auto desc_mn = [&](uint32_t buf, uint32_t panel, int k) {
                return smem_desc_sw128(sbase + buf + (uint32_t)k * 2048u, panel, 1024u);
            };
            const uint32_t tile0 = blockIdx.x;
            mbar_expect_tx(&x_full[0], 8192);
            tma_load_2d(smem + kX, &tmap_x, 0, (int32_t)(tile0 * NS), &x_full[0]);
            mbar_expect_tx(t_full, 8192);
            tma_load_2d(smem + kDZ4, &tmap_t, 0, (int32_t)(tile0 * NS), t_full);
            uint32_t x_issued = 1, t_issued = 1;  // loads issued so far (for the drain after an abort)

            for (uint32_t it = 0; it < n_my_tiles && ok; ++it) {
                const uint32_t b = it & 1u;
                const uint32_t next_tile = blockIdx.x + (it + 1) * gridDim.x;
                const bool has_next = it + 1 < n_my_tiles;
                const uint32_t xbuf = kX + b * 8192u;
                // ---- forward ----
                acc_wait();
                if (!ok) break;
                if (has_next) {  // the other X buffer was last read by the previous tile's dW_0 product, now complete
                    mbar_expect_tx(&x_full[b ^ 1u], 8192);
                    tma_load_2d(smem + kX + (b ^ 1u) * 8192u, &tmap_x, 0, (int32_t)(next_tile * NS), &x_full[b ^ 1u]);
                    ++x_issued;
                }
                ok = mbar_wait(&x_full[b], (it >> 1) & 1u, abort_flag, p.status, kStatusCtrlX);
                if (!ok) break;
                for (int k = 0; k < D0 / 16; ++k)
                    umma_f16(acc, desc_k(kW0, 16384u, k), desc_k(xbuf, 8192u, k), kIdescFwd, k > 0);
                umma_commit(acc_full);
                ++step;
                for (int l = 1; l < NL && ok; ++l) {
                    acc_wait();
                    if (!ok) break;
                    const uint32_t wpanel = (uint32_t)out_dim(l) * 128u;
                    const uint32_t abuf = kA1 + (uint32_t)(l - 1) * 16384u;
                    for (int k = 0; k < H / 16; ++k)
                        umma_f16(acc, desc_k(w_off(l), wpanel, k), desc_k(abuf, 8192u, k), kIdescFwd, k > 0);
                    umma_commit(acc_full);
                    ++step;
                }
                // ---- backward ----
                for (int l = NL - 1; l >= 1 && ok; --l) {
                    acc_wait();
                    if (!ok) break;
                    if (l == NL - 2 && has_next) {  // dZ_4's buffer is free: fetch the next tile's targets
                        mbar_expect_tx(t_full, 8192);
                        tma_load_2d(smem + kDZ4, &tmap_t, 0, (int32_t)(next_tile * NS), t_full);
                        ++t_issued;
                    }
                    const uint32_t wpanel = (uint32_t)out_dim(l) * 128u;
                    const uint32_t dzbuf = (l == NL - 1) ? kDZ4 : kA1 + (uint32_t)l * 16384u;  // dZ_l lives in A_{l+1}'s buffer
                    const uint32_t abuf = kA1 + (uint32_t)(l - 1) * 16384u;                   // A_l
                    const int kdx = out_dim(l) / 16;
                    for (int k = 0; k < kdx; ++k)
                        umma_f16(acc, desc_mn(w_off(l), wpanel, k), desc_k(dzbuf, 8192u, k), kIdescDx, k > 0);
                    if (l == NL - 1) {
                        for (int k = 0; k < NS / 16; ++k)
                            umma_f16(tmem_base + kColDW4T, desc_mn(abuf, 8192u, k), desc_mn(dzbuf, 8192u, k), kIdescDw64,
                                     (it > 0 || k > 0));
                    } else {
                        for (int k = 0; k < NS / 16; ++k)
                            umma_f16(tmem_base + kColDW1 + (uint32_t)(l - 1) * 128u, desc_mn(dzbuf, 8192u, k),
                                     desc_mn(abuf, 8192u, k), kIdescDw, (it > 0 || k > 0));
                    }
                    umma_commit(acc_full);
                    ++step;
                }
                if (!ok) break;
                // ---- dW_0 into the shared accumulator; the epilogue adds it to registers ----
                acc_wait();
                if (!ok) break;
                for (int k = 0; k < NS / 16; ++k)
                    umma_f16(acc, desc_mn(kA1, 8192u, k), desc_mn(xbuf, 8192u, k), kIdescDw64, k > 0);
                umma_commit(acc_full);
                ++step;
            }
            if (*abort_flag) {
                // Give the copies still in flight a bounded time to land before the CTA exits.
                if (x_issued > 0) mbar_drain(&x_full[(x_issued - 1) & 1u], ((x_issued - 1) >> 1) & 1u);
                if (t_issued > 0) mbar_drain(t_full, (t_issued - 1) & 1u);
            }
        }
    } else if (warp >= 2) {
        // =================================== epilogue warps ========================================
        const int q = warp & 3;                // TMEM lane quarter this warp may read
        const int h = (warp - 2) >> 2;         // which half of the 64 sample columns
        const int f = q * 32 + lane;           // the feature (TMEM lane) this thread owns
        const int col0 = h * 32;
        const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + kColAcc + (uint32_t)col0;
        // Byte offset of (row col0, feature f) inside a [64 x W] operand buffer, minus the swizzled chunk.
        const uint32_t pbase = (uint32_t)(f >> 6) * 8192u + (uint32_t)col0 * 128u + (uint32_t)(f & 7) * 2u;
        uint32_t xo[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) xo[j] = pbase + (uint32_t)(((((f & 63) >> 3) ^ j)) << 4);

        float bias[NL];
#pragma unroll
        for (int l = 0; l < NL; ++l) bias[l] = s_bias[l * 128 + f];
        uint32_t dreg[NL - 1][16];   // activation derivatives of the four hidden layers, two per register
        float dw0[32];               // this thread's slice of dW_0 (row f, columns col0..col0+31), summed over tiles
        float db[NL];                // bias-gradient partial sums
#pragma unroll
        for (int i = 0; i < 32; ++i) dw0[i] = 0.0f;
#pragma unroll
        for (int l = 0; l < NL; ++l) db[l] = 0.0f;
        float run_max = 0.0f, run_sum = 0.0f;
        uint32_t step = 0;
        bool ok = true;

        auto release_acc = [&]() {
            tc_fence_before();
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_free);
        };

        for (uint32_t it = 0; it < n_my_tiles && ok; ++it) {
            const uint32_t tile = blockIdx.x + it * gridDim.x;
            // ---- forward, hidden layers ----
#pragma unroll
            for (int l = 0; l < NL - 1; ++l) {
                ok = ok && mbar_wait(acc_full, step & 1u, abort_flag, p.status, kStatusEpiAcc);
                ++step;
                if (!ok) break;
                tc_fence_after();
                uint32_t v[32];
                tmem_ld_32x32(t_acc, v);
                tmem_ld_wait();
                uint8_t* dst = smem + kA1 + (uint32_t)l * 16384u;
#pragma unroll
                for (int s = 0; s < 32; s += 2) {
                    float a0, d0, a1, d1;
                    act_pair<ACT>(E::round(__uint_as_float(v[s]) + bias[l]), p.act_alpha, a0, d0);
                    act_pair<ACT>(E::round(__uint_as_float(v[s + 1]) + bias[l]), p.act_alpha, a1, d1);
                    *(uint16_t*)(dst + xo[s & 7] + s * 128) = E::pack(a0);
                    *(uint16_t*)(dst + xo[(s + 1) & 7] + (s + 1) * 128) = E::pack(a1);
                    dreg[l][s >> 1] = (uint32_t)E::pack(d0) | ((uint32_t)E::pack(d1) << 16);
                }
                release_acc();
            }
            if (!ok) break;
            // ---- output layer, loss and dZ_4 ----
            {
                ok = ok && mbar_wait(acc_full, step & 1u, abort_flag, p.status, kStatusEpiAcc);
                ++step;
                ok = ok && mbar_wait(t_full, it & 1u, abort_flag, p.status, kStatusEpiTarget);
                if (!ok) break;
                tc_fence_after();
                if (q < 2) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_acc, v);
                    tmem_ld_wait();
                    uint8_t* dst = smem + kDZ4;
                    float lsq[32];
#pragma unroll
                    for (int s = 0; s < 32; ++s) {
                        const bool valid = tile * NS + col0 + s < p.count;
                        uint16_t* slot = (uint16_t*)(dst + xo[s & 7] + s * 128);
                        const float out = E::round(__uint_as_float(v[s]) + bias[NL - 1]);
                        const float diff = out - E::unpack(*slot);
                        const float dz = valid ? E::round((2.0f * p.loss_scale) * diff) : 0.0f;
                        lsq[s] = valid ? (diff * p.loss_scale) * diff : 0.0f;
                        *slot = E::pack(dz);
                        db[NL - 1] += dz;
                    }
                    // Sum over this warp's 32 features for each of the 32 sample columns: after the
                    // five exchange rounds lane c holds the sum of column c.
#pragma unroll
                    for (int w = 16; w >= 1; w >>= 1) {
                        const bool upper = (lane & w) != 0;
#pragma unroll
                        for (int i = 0; i < w; ++i) {
                            const float keep = upper ? lsq[i + w] : lsq[i];
                            const float send = upper ? lsq[i] : lsq[i + w];
                            lsq[i] = keep + __shfl_xor_sync(0xffffffffu, send, w);
                        }
                    }
                    s_loss_part[q * 64 + col0 + lane] = lsq[0];
                    __syncwarp();
                    if (lane == 0) mbar_arrive(loss_bar);
                }
                release_acc();
                if (q == 0) {
                    // The other feature half of these 32 samples comes from the warp of quarter 1.
                    ok = ok && mbar_wait(loss_bar, it & 1u, abort_flag, p.status, kStatusEpiLoss);
                    if (!ok) break;
                    float tot = s_loss_part[col0 + lane] + s_loss_part[64 + col0 + lane];
                    float mx = tot;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                        tot += __shfl_xor_sync(0xffffffffu, tot, o);
                    }
                    run_max = fmaxf(run_max, mx);
                    run_sum += tot;
                }
            }
            // ---- backward: dA_l arrives in the accumulator, dZ_{l-1} replaces A_l in shared memory ----
#pragma unroll
            for (int l = NL - 1; l >= 1; --l) {
                ok = ok && mbar_wait(acc_full, step & 1u, abort_flag, p.status, kStatusEpiAcc);
                ++step;
                if (!ok) break;
                tc_fence_after();
                uint32_t v[32];
                tmem_ld_32x32(t_acc, v);
                tmem_ld_wait();
                uint8_t* dst = smem + kA1 + (uint32_t)(l - 1) * 16384u;
#pragma unroll
                for (int s = 0; s < 32; s += 2) {
                    const uint32_t dd = dreg[l - 1][s >> 1];
                    const float dz0 = E::round(__uint_as_float(v[s]) * E::unpack((uint16_t)(dd & 0xffffu)));
                    const float dz1 = E::round(__uint_as_float(v[s + 1]) * E::unpack((uint16_t)(dd >> 16)));
                    *(uint16_t*)(dst + xo[s & 7] + s * 128) = E::pack(dz0);
                    *(uint16_t*)(dst + xo[(s + 1) & 7] + (s + 1) * 128) = E::pack(dz1);
                    db[l - 1] += dz0 + dz1;
                }
                release_acc();
            }
            if (!ok) break;
            // ---- dW_0 of this tile: add the accumulator to the register slice ----
            {
                ok = ok && mbar_wait(acc_full, step & 1u, abort_flag, p.status, kStatusEpiAcc);
                ++step;
                if (!ok) break;
                tc_fence_after();
                uint32_t v[32];
                tmem_ld_32x32(t_acc, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) dw0[i] += __uint_as_float(v[i]);
                release_acc();
            }
        }

        // ---- one add per parameter per CTA ----
        if (ok && !*abort_flag && n_my_tiles > 0) {
            tc_fence_after();
            const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
            for (int l = 1; l <= 3; ++l) {
                float* dW = (float*)p.net[l].weightsGrad + (size_t)f * 128;
                for (int c = 0; c < 2; ++c) {
                    const int col = h * 64 + c * 32;
                    uint32_t v[32];
                    tmem_ld_32x32(lane_base + kColDW1 + (uint32_t)(l - 1) * 128u + (uint32_t)col, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) atomicAdd(dW + col + i, __uint_as_float(v[i]));
                }
            }
            {
                // dW_4^T: lane = input feature, column = output feature.
                float* dW = (float*)p.net[4].weightsGrad;
                uint32_t v[32];
                tmem_ld_32x32(lane_base + kColDW4T + (uint32_t)col0, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) atomicAdd(dW + (size_t)(col0 + i) * 128 + f, __uint_as_float(v[i]));
            }
            {
                float* dW = (float*)p.net[0].weightsGrad + (size_t)f * 64 + col0;
#pragma unroll
                for (int i = 0; i < 32; ++i) atomicAdd(dW + i, dw0[i]);
            }
#pragma unroll
            for (int l = 0; l < NL; ++l)
                if (l < NL - 1 || f < DOUT) atomicAdd((float*)p.net[l].biasesGrad + f, db[l]);
            if (q == 0 && lane == 0) {
                atomicMax(p.loss_words, __float_as_uint(run_max));
                atomicAdd((float*)(p.loss_words + 1), run_sum);
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
// Host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct TcWorkspace {
    int ordinal = 0;
    int sm_count = 0;
    uint32_t* status = nullptr;       // device word, set by kernels that give up on a wait
    uint32_t* status_host = nullptr;  // pinned copy
    EncodeTiledFn encode = nullptr;
};

bool tc_forward_supported(const MlpConfig&) { return false; }

bool tc_train_supported(const MlpConfig& c)
{
    static const int dims[6] = {64, 128, 128, 128, 128, 64};
    if (c.n_layers != 5) return false;
    for (int i = 0; i < 6; ++i)
        if (c.dims[i] != dims[i]) return false;
    if (c.dtype != MLP_BF16 && c.dtype != MLP_F16) return false;
    if (c.input_dtype != c.dtype || c.target_dtype != c.dtype) return false;
    if (c.hidden_act != MLP_ACT_GELU_TANH && c.hidden_act != MLP_ACT_RELU && c.hidden_act != MLP_ACT_LEAKY_RELU) return false;
    if (c.output_act != MLP_ACT_IDENTITY || c.encoding != MLP_ENC_NONE) return false;
    return true;
}

TcWorkspace* tc_workspace_create(int ordinal, std::string* err)
{
    TcWorkspace* ws = new TcWorkspace();
    ws->ordinal = ordinal;
    cudaError_t e = cudaDeviceGetAttribute(&ws->sm_count, cudaDevAttrMultiProcessorCount, ordinal);
    if (e == cudaSuccess) e = cudaMalloc((void**)&ws->status, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ws->status, 0, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMallocHost((void**)&ws->status_host, sizeof(uint32_t));
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
    delete ws;
}

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

// A [rows][cols] 16-bit row-major matrix viewed in boxes of box_rows x 64 columns with the 128-byte swizzle.
static bool make_tile_map(TcWorkspace* ws, CUtensorMap* map, int dtype, uint64_t base, uint64_t rows, uint32_t cols,
                          uint32_t box_rows, std::string* err)
{
    if (base & 15u) { if (err) *err = "inputs and targets must be 16-byte aligned for the TMA path"; return false; }
    const cuuint64_t gdim[2] = {cols, rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = ws->encode(map, dtype == MLP_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                            (void*)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { if (err) *err = "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r); return false; }
    return true;
}

template <int FMT, int ACT>
static cudaError_t launch_wide(cudaStream_t st, TcWorkspace* ws, const CUtensorMap& mx, const CUtensorMap& mt,
                               const WideTrainParams& p)
{
    auto kern = learn_gradient_wide_kernel<FMT, ACT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wide::kSmemBytes);
    if (e != cudaSuccess) return e;
    const uint32_t grid = p.n_tiles < (uint32_t)ws->sm_count ? p.n_tiles : (uint32_t)ws->sm_count;
    kern<<<grid, wide::kThreads, wide::kSmemBytes, st>>>(mx, mt, p);
    return cudaGetLastError();
}

cudaError_t launch_learn_gradient_tc(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const MlpLearnGradParamsEx& a,
                                     int* launches, std::string* err)
{
    if (!tc_train_supported(c)) { if (err) *err = "shape not built for the tensor-core path"; return cudaErrorInvalidValue; }
    if (a.count == 0) return cudaSuccess;
    CUtensorMap mx, mt;
    if (!make_tile_map(ws, &mx, c.dtype, a.inputs, a.count, 64, wide::NS, err)) return cudaErrorInvalidValue;
    if (!make_tile_map(ws, &mt, c.dtype, a.targets, a.count, 64, wide::NS, err)) return cudaErrorInvalidValue;
    WideTrainParams p;
    p.net = (const MlpLayerPointers*)a.networkBuffer;
    p.loss_words = (uint32_t*)a.lossBuffer;
    p.status = ws->status;
    p.count = a.count;
    p.n_tiles = (a.count + wide::NS - 1) / wide::NS;
    p.loss_scale = c.loss == MLP_LOSS_MSE_MEAN ? 1.0f / 64.0f : 1.0f;
    p.act_alpha = c.act_alpha;
    cudaError_t e = cudaErrorInvalidValue;
#define MLPB200_DISPATCH(FMT_, ACT_) \
    if (c.dtype == FMT_ && c.hidden_act == ACT_) e = launch_wide<FMT_, ACT_>(st, ws, mx, mt, p);
    MLPB200_DISPATCH(MLP_BF16, MLP_ACT_GELU_TANH)
    MLPB200_DISPATCH(MLP_BF16, MLP_ACT_RELU)
    MLPB200_DISPATCH(MLP_BF16, MLP_ACT_LEAKY_RELU)
    MLPB200_DISPATCH(MLP_F16, MLP_ACT_GELU_TANH)
    MLPB200_DISPATCH(MLP_F16, MLP_ACT_RELU)
    MLPB200_DISPATCH(MLP_F16, MLP_ACT_LEAKY_RELU)
#undef MLPB200_DISPATCH
    *launches += 1;
    return e;
}

cudaError_t launch_forward_tc(cudaStream_t, TcWorkspace*, const MlpConfig&, const MlpForwardParams&, int*, std::string* err)
{
    if (err) *err = "no tensor-core forward kernel for this shape";
    return cudaErrorInvalidValue;
}

}  // namespace mlpb200
