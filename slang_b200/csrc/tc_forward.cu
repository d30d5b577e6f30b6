// Forward-only MLP on the tensor cores (tcgen05 / TMEM / TMA) for sm_100a: the inference sweep
// (depth-4 networks of constant width 16..128, 16-bit weights, fp32 outputs) and any network whose
// widths are DIN -> DH -> ... -> DH -> DOUT with every width in {16, 32, 64, 128}.
//
// Orientation: samples run along the 128 TMEM lanes (the MMA's M), features along the columns:
//   Z_l [128 x out] = A_l [128 x in] . W_l^T        A: activations, K-major      B: W_l [out][in], K-major
// An epilogue thread owns one sample row: it reads the row's accumulator columns, adds the bias,
// applies the activation and writes the row of the next layer's operand as 16-byte chunks (or, after
// the last layer, the fp32 outputs to global memory).  Several 128-sample tiles ("chains") are in
// flight per CTA, each with its own accumulator columns, operand buffer and four epilogue warps, so
// that one chain's epilogue overlaps another chain's products and input loads: at small widths the
// work per tile is tiny and only concurrency hides the hand-off latencies.
//
// Operand layout: rows of min(64, width) elements per panel with the swizzle whose span equals the
// panel row (32, 64 or 128 bytes), which is exactly what a TMA tile load with that swizzle produces.
//
// What the reference does instead: one thread per sample with scalar loops (coopVecMatMulAdd's
// fallback, source/slang/hlsl.meta.slang:32835-32912) or one warp per 32 samples on mma.sync with
// shuffle-packed operands (source/standard-modules/neural/mma-tiled-cuda.slang:88-138).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string>

#include "launchers.h"
#include "mlp_common.cuh"
#include "tc_host.h"
#include "tc_layout.cuh"
#include "tc_ptx.cuh"

namespace mlpb200 {

using namespace ptx;

namespace fwd {

using namespace layout;

enum : uint32_t { kStatusCtrlX = 0x100u, kStatusCtrlAcc = 0x200u, kStatusEpiAcc = 0x400u, kStatusAlign = 0x800u };

struct Params {
    const MlpLayerPointers* net;
    float* out;
    uint32_t* status;
    uint32_t count;
    uint32_t n_tiles;
    float act_alpha;
    uint32_t out_storage;  // 1: outputs are written in the network's 16-bit storage type instead of fp32
    int param_layout;      // MlpParamLayout of the weights
};

template <int FMT> struct Cvt;
template <> struct Cvt<MLP_BF16> {
    __device__ static __forceinline__ float lo(uint32_t p) { return __uint_as_float(p << 16); }
    __device__ static __forceinline__ float hi(uint32_t p) { return __uint_as_float(p & 0xffff0000u); }
    // max(x, 0) on both halves of a packed pair (exact: rounding is monotonic and zero is representable)
    __device__ static __forceinline__ uint32_t relu2(uint32_t p)
    {
        __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&p);
        v = __hmax2(v, __float2bfloat162_rn(0.0f));
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __device__ static __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi)
    {
        __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&t);
    }
};
template <> struct Cvt<MLP_F16> {
    __device__ static __forceinline__ float lo(uint32_t p) { return __half2float(__ushort_as_half((uint16_t)(p & 0xffffu))); }
    __device__ static __forceinline__ float hi(uint32_t p) { return __half2float(__ushort_as_half((uint16_t)(p >> 16))); }
    __device__ static __forceinline__ uint32_t relu2(uint32_t p)
    {
        __half2 v = *reinterpret_cast<__half2*>(&p);
        v = __hmax2(v, __float2half2_rn(0.0f));
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __device__ static __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi)
    {
        __half2 t = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&t);
    }
};

template <int DIN, int DH, int DOUT, int NL, int NCH, int CS>
struct Geometry {
    static constexpr int kThreads = 64 + 128 * NCH * CS;  // CS: warps sharing a lane quarter split the columns
    static constexpr int kAccCols = imax(DH, DOUT);
    static constexpr uint32_t kTmemCols = pow2_at_least_32(NCH * kAccCols);
    __host__ __device__ static constexpr int in_dim(int l) { return l == 0 ? DIN : DH; }
    __host__ __device__ static constexpr int out_dim(int l) { return l == NL - 1 ? DOUT : DH; }
    __host__ __device__ static constexpr uint32_t w_bytes(int l) { return (uint32_t)(in_dim(l) * out_dim(l) * 2); }
    __host__ __device__ static constexpr uint32_t w_off(int l)
    {
        uint32_t o = 0;
        for (int i = 0; i < l; ++i) o += (w_bytes(i) + 1023u) & ~1023u;
        return o;
    }
    static constexpr uint32_t kActBytes = (uint32_t)(128 * imax(DIN, DH) * 2 + 1023) & ~1023u;
    static constexpr uint32_t kAct = w_off(NL);
    // fp32 output staging per chain: slabs of [128 rows][kSlabCols floats] in the layout of a swizzled TMA store
    static constexpr int kSlabCols = DOUT < 32 ? DOUT : (DH >= 128 ? 16 : 32);  // narrower slabs where the weights fill shared memory
    static constexpr uint32_t kStageBytes = 128u * kSlabCols * 4u;
    static constexpr uint32_t kStage = kAct + NCH * kActBytes;
    static constexpr uint32_t kBias = kStage + NCH * CS * kStageBytes;  // fp32 [NL][128]
    static constexpr uint32_t kBars = kBias + NL * 128 * 4;        // x_full, acc_full, acc_free, stg_full, stg_free (NCH each)
    static constexpr uint32_t kTmemPtr = kBars + (3 + 2 * CS) * NCH * 8;
    static constexpr uint32_t kAbort = kTmemPtr + 4;
    static constexpr uint32_t kSmemBytes = kAbort + 4;  // the dynamic shared-memory base must be 1024-byte aligned (checked at run time)
    static_assert((DH / CS) % 16 == 0 && (DOUT / CS) % 16 == 0, "column split");
};

// CPS: CTAs per SM the build is sized for (the narrow widths run three CTAs of two chains each: three control
// warps walk their chains independently).
// NCW: control warps (1 or 2).
template <int DIN, int DH, int DOUT, int NL, int FMT, int ACT, int OUT_ACT, int NCH, int CS, int CPS = 1, int NCW = 1>
__global__ void __launch_bounds__(64 + 128 * NCH * CS, CPS)
forward_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_out, const Params p)
{
    using G = Geometry<DIN, DH, DOUT, NL, NCH, CS>;
    using C = Cvt<FMT>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    const uint32_t sbase = smem_u32(smem);
    if (sbase & 1023u) {  // the swizzled operand layouts need a 1024-byte aligned base
        if (threadIdx.x == 0) atomicOr(p.status, kStatusAlign);
        return;
    }
    uint64_t* x_full = (uint64_t*)(smem + G::kBars);
    uint64_t* acc_full = x_full + NCH;
    uint64_t* acc_free = acc_full + NCH;
    uint64_t* stg_full = acc_free + NCH;   // the chain's four warps have written the output slab
    uint64_t* stg_free = stg_full + NCH * CS;  // the slab's TMA store has finished reading shared memory
    uint32_t* tmem_ptr = (uint32_t*)(smem + G::kTmemPtr);
    volatile uint32_t* abort_flag = (volatile uint32_t*)(smem + G::kAbort);
    float* s_bias = (float*)(smem + G::kBias);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n_my_tiles = (p.n_tiles > blockIdx.x) ? (p.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    constexpr uint32_t kXBytes = 128u * DIN * 2u;

    if (threadIdx.x == 0) {
        for (int c = 0; c < NCH; ++c) {
            mbar_init(&x_full[c], 1);
            mbar_init(&acc_full[c], 1);
            mbar_init(&acc_free[c], 4 * CS);
        }
        for (int c = 0; c < NCH * CS; ++c) {
            mbar_init(&stg_full[c], 4);
            mbar_init(&stg_free[c], 1);
        }
        *abort_flag = 0u;
        fence_mbar_init();
        prefetch_tmap(&tmap_x);
        prefetch_tmap(&tmap_out);
    }
    if (warp == 1) {
        tmem_alloc(tmem_ptr, G::kTmemCols);
        tmem_relinquish();
    }
    // Weights into shared memory, row-major rows re-cut into swizzled panels; biases as fp32.
    for (int l = 0; l < NL; ++l) {
        const int in = G::in_dim(l), out = G::out_dim(l);
        const uint4* src = (const uint4*)p.net[l].weights;
        const uint16_t* src16 = (const uint16_t*)p.net[l].weights;
        const int cpr = in / 8;
        for (int idx = threadIdx.x; idx < out * cpr; idx += G::kThreads) {
            const int o = idx / cpr, j = idx % cpr;
            const uint32_t off = (l == 0) ? chunk_offset<DIN>(out, o, j) : chunk_offset<DH>(out, o, j);
            uint4 v;
            if (p.param_layout == MLP_PARAMS_ROW_MAJOR) {
                v = src[idx];
            } else {
                // OptimalLayout: the eight inputs of a chunk are four pairs inside one 16x16 tile
                uint16_t hw[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) hw[e] = src16[weight_index(MLP_PARAMS_OPTIMAL, in, out, o, j * 8 + e)];
                v = make_uint4(hw[0] | ((uint32_t)hw[1] << 16), hw[2] | ((uint32_t)hw[3] << 16), hw[4] | ((uint32_t)hw[5] << 16),
                               hw[6] | ((uint32_t)hw[7] << 16));
            }
            *(uint4*)(smem + G::w_off(l) + off) = v;
        }
        for (int j = threadIdx.x; j < 128; j += G::kThreads)
            s_bias[l * 128 + j] = j < out ? load_as_f32(FMT, (const void*)p.net[l].biases, j) : 0.0f;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    // The i-th tile of this CTA (global tile blockIdx.x + i * gridDim.x) runs on chain i % NCH.
    if (warp < NCW) {
        // =================================== control warps =========================================
        // With two of them, warp w walks the chains w, w + 2, ... in lock step among themselves only, so a
        // chain that is late holds up at most half of the others (measured: +9 % at width 64, a loss at
        // widths 16 and 128).  (Warp 1 also owns the tensor-memory allocation.)
        if (n_my_tiles > 0) {
            const int cw = warp;
            const bool leader = elect_one();
            constexpr uint32_t F = FMT == MLP_BF16 ? 1u : 0u;
            const uint32_t lo_base = (sbase & 0x3FFFFu) >> 4;
            bool ok = true;
            uint32_t steps[NCH];  // products issued so far per chain
#pragma unroll
            for (int c = 0; c < NCH; ++c) steps[c] = 0;
            if (leader) {
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    if (c % NCW == cw && (uint32_t)c < n_my_tiles) {
                        const uint32_t tile = blockIdx.x + (uint32_t)c * gridDim.x;
                        mbar_expect_tx(&x_full[c], kXBytes);
#pragma unroll
                        for (int pn = 0; pn < DIN / panel_w(DIN); ++pn)
                            tma_load_2d(smem + G::kAct + c * G::kActBytes + pn * (128 * row_bytes(DIN)), &tmap_x, pn * panel_w(DIN),
                                        (int32_t)(tile * 128u), &x_full[c]);
                    }
                }
            }
            const uint32_t rounds = (n_my_tiles + NCH - 1) / NCH;
            for (uint32_t j = 0; j < rounds && ok; ++j) {
#pragma unroll
                for (int l = 0; l < NL; ++l) {
#pragma unroll
                    for (int c = 0; c < NCH; ++c) {
                        if (c % NCW == cw && j * NCH + c < n_my_tiles && ok) {
                            // Every phase of the chain's barriers is observed in order.
                            if (steps[c] > 0) ok = mbar_wait(&acc_free[c], (steps[c] - 1) & 1u, abort_flag, p.status, kStatusCtrlAcc);
                            if (l == 0) ok = ok && mbar_wait(&x_full[c], j & 1u, abort_flag, p.status, kStatusCtrlX);
                            tc_fence_after();
                            if (ok) {
                                const uint32_t acc = tmem_base + (uint32_t)(c * G::kAccCols);
                                const uint32_t abuf = G::kAct + (uint32_t)c * G::kActBytes;
                                if (leader) {
                                    if (l == 0) {
                                        constexpr uint32_t hi = (uint32_t)((8 * row_bytes(DIN)) >> 4) | (1u << 14) | (layout_type(DIN) << 29);
                                        constexpr uint32_t idesc = umma_idesc(F, 0, 0, 128, G::out_dim(0));
#pragma unroll
                                        for (int k = 0; k < DIN / 16; ++k) {
                                            constexpr int kpp = panel_w(DIN) / 16;  // K steps per panel
                                            const uint32_t ka = (uint32_t)(k / kpp) * (uint32_t)(128 * row_bytes(DIN)) + (uint32_t)(k % kpp) * 32u;
                                            const uint32_t kb = (uint32_t)(k / kpp) * (uint32_t)(G::out_dim(0) * row_bytes(DIN)) + (uint32_t)(k % kpp) * 32u;
                                            const uint64_t da = ((uint64_t)hi << 32) | (lo_base + ((abuf + ka) >> 4) + (1u << 16));
                                            const uint64_t db = ((uint64_t)hi << 32) | (lo_base + ((G::w_off(0) + kb) >> 4) + (1u << 16));
                                            umma_f16(acc, da, db, idesc, k > 0);
                                        }
                                    } else {
                                        constexpr uint32_t hi = (uint32_t)((8 * row_bytes(DH)) >> 4) | (1u << 14) | (layout_type(DH) << 29);
                                        const uint32_t idesc = umma_idesc(F, 0, 0, 128, G::out_dim(l));
#pragma unroll
                                        for (int k = 0; k < DH / 16; ++k) {
                                            constexpr int kpp = panel_w(DH) / 16;
                                            const uint32_t ka = (uint32_t)(k / kpp) * (uint32_t)(128 * row_bytes(DH)) + (uint32_t)(k % kpp) * 32u;
                                            const uint32_t kb = (uint32_t)(k / kpp) * (uint32_t)(G::out_dim(l) * row_bytes(DH)) + (uint32_t)(k % kpp) * 32u;
                                            const uint64_t da = ((uint64_t)hi << 32) | (lo_base + ((abuf + ka) >> 4) + (1u << 16));
                                            const uint64_t db = ((uint64_t)hi << 32) | (lo_base + ((G::w_off(l) + kb) >> 4) + (1u << 16));
                                            umma_f16(acc, da, db, idesc, k > 0);
                                        }
                                    }
                                    umma_commit(&acc_full[c]);
                                }
                                __syncwarp();
                                ++steps[c];
                            }
                        }
                    }
                }
            }
        }
    } else if (warp >= 2) {
        // =================================== epilogue warps ========================================
        const int g = (warp - 2) >> 2;   // group of four warps: one chain's share of the columns
        const int c = g / CS;            // chain
        const int sub = g % CS;          // which part of the layer's columns
        const int q = warp & 3;          // TMEM lane quarter this warp may read
        const int r = q * 32 + lane;     // the sample row this thread owns
        const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * G::kAccCols);
        uint8_t* abuf = smem + G::kAct + c * G::kActBytes;
        uint8_t* stage = smem + G::kStage + g * G::kStageBytes;
        uint32_t step = 0, slabs = 0;  // slabs: output slabs this chain has handed to TMA stores so far
        bool ok = true;
        for (uint32_t i = (uint32_t)c; i < n_my_tiles && ok; i += NCH) {
            const uint32_t tile = blockIdx.x + i * gridDim.x;
#pragma unroll
            for (int l = 0; l < NL; ++l) {
                ok = ok && mbar_wait(&acc_full[c], step & 1u, abort_flag, p.status, kStatusEpiAcc);
                ++step;
                if (ok) {
                    tc_fence_after();
                    const bool last = (l == NL - 1);
                    if (last && sub == 0 && q == 0 && lane == 0 && i + NCH < n_my_tiles) {
                        // The last product has read this chain's operand buffer: fetch the chain's next tile.
                        const uint32_t next = blockIdx.x + (i + NCH) * gridDim.x;
                        mbar_expect_tx(&x_full[c], kXBytes);
#pragma unroll
                        for (int pn = 0; pn < DIN / panel_w(DIN); ++pn)
                            tma_load_2d(abuf + pn * (128 * row_bytes(DIN)), &tmap_x, pn * panel_w(DIN), (int32_t)(next * 128u), &x_full[c]);
                    }
                    const int out = G::out_dim(l);
                    const float* bl = s_bias + l * 128;
                    const uint64_t row_index = (uint64_t)tile * 128u + (uint64_t)r;
                    // The accumulator is read 16 columns at a time, one read ahead: the next piece's read is issued
                    // as soon as the current piece has arrived and runs under the current piece's arithmetic.
                    const int kPieces = G::out_dim(l) / CS / 16;
                    uint32_t vbuf[2][16];
                    tmem_ld_32x16(t_acc + (uint32_t)(sub * (G::out_dim(l) / CS)), vbuf[0]);
#pragma unroll
                    for (int pc = 0; pc < kPieces; ++pc) {
                        const int cc = pc * 16;
                        const int c0 = sub * (G::out_dim(l) / CS) + cc;  // this warp's share of the columns
                        uint32_t (&v)[16] = vbuf[pc & 1];
                        tmem_ld_wait();
                        if (pc + 1 < kPieces) tmem_ld_32x16(t_acc + (uint32_t)(c0 + 16), vbuf[(pc + 1) & 1]);
                        // bias (packed fp32 adds) and rounding to the storage type, two values per register
                        uint32_t zp[8];
#pragma unroll
                        for (int k = 0; k < 16; k += 4) {
                            const float4 b4 = *(const float4*)(bl + c0 + k);
                            const float2 s0 = __fadd2_rn(make_float2(__uint_as_float(v[k]), __uint_as_float(v[k + 1])), make_float2(b4.x, b4.y));
                            const float2 s1 = __fadd2_rn(make_float2(__uint_as_float(v[k + 2]), __uint_as_float(v[k + 3])), make_float2(b4.z, b4.w));
                            zp[k >> 1] = C::pack2(s0.x, s0.y);
                            zp[(k >> 1) + 1] = C::pack2(s1.x, s1.y);
                        }
                        if (!last) {
                            uint32_t pk[8];
                            if constexpr (ACT == MLP_ACT_RELU) {
#pragma unroll
                                for (int k = 0; k < 8; ++k) pk[k] = C::relu2(zp[k]);
                            } else {
#pragma unroll
                                for (int k = 0; k < 8; ++k)
                                    pk[k] = C::pack2(act_value(ACT, p.act_alpha, C::lo(zp[k])), act_value(ACT, p.act_alpha, C::hi(zp[k])));
                            }
                            // the next layer reads this buffer as a [128][DH] operand
                            *(uint4*)(abuf + chunk_offset<DH>(128, r, c0 / 8)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            *(uint4*)(abuf + chunk_offset<DH>(128, r, c0 / 8 + 1)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                        } else {
                            if (p.out_storage) {
                              if (row_index < p.count) {
                                uint32_t pk[8];
#pragma unroll
                                for (int k = 0; k < 8; ++k)
                                    pk[k] = (OUT_ACT == MLP_ACT_IDENTITY) ? zp[k]
                                            : C::pack2(act_value(OUT_ACT, p.act_alpha, C::lo(zp[k])), act_value(OUT_ACT, p.act_alpha, C::hi(zp[k])));
                                uint4* dst = (uint4*)((uint16_t*)p.out + row_index * (uint64_t)out + c0);
                                dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                                dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                              }
                            } else {
                                // fp32 outputs go through a staging slab and a TMA store: every 128-byte line
                                // of the output is written once, whole (rows past the batch are clipped by the copy)
                                constexpr int SC = G::kSlabCols;          // columns per slab
                                constexpr int CPR = SC / 4;               // 16-byte chunks per slab row
                                const int cs = c0 % SC;                   // first column of this 16-column piece inside the slab
                                if (cs == 0) {
                                    if (slabs > 0) ok = ok && mbar_wait(&stg_free[g], (slabs - 1) & 1u, abort_flag, p.status, kStatusEpiAcc);
                                }
#pragma unroll
                                for (int k = 0; k < 8; k += 2) {
                                    const int chunk = (cs + 2 * k) / 4;
                                    const int sw = SC == 32 ? (r & 7) : SC == 16 ? ((r >> 1) & 3) : 0;
                                    *(float4*)(stage + (uint32_t)r * (SC * 4) + (uint32_t)(((chunk ^ sw) % CPR) << 4)) =
                                        make_float4(act_value(OUT_ACT, p.act_alpha, C::lo(zp[k])), act_value(OUT_ACT, p.act_alpha, C::hi(zp[k])),
                                                    act_value(OUT_ACT, p.act_alpha, C::lo(zp[k + 1])), act_value(OUT_ACT, p.act_alpha, C::hi(zp[k + 1])));
                                }
                                if (cs + 16 >= SC) {
                                    // the slab is complete in this warp: hand it over, one lane of the chain stores it
                                    fence_async_smem();
                                    __syncwarp();
                                    if (lane == 0) mbar_arrive(&stg_full[g]);
                                    if (q == 0 && lane == 0) {
                                        ok = ok && mbar_wait(&stg_full[g], slabs & 1u, abort_flag, p.status, kStatusEpiAcc);
                                        if (ok) {
                                            tma_store_2d(&tmap_out, (c0 / SC) * SC, (int32_t)(tile * 128u), stage);
                                            tma_store_commit();
                                            tma_store_wait_read();
                                            mbar_arrive(&stg_free[g]);
                                        }
                                    }
                                    ++slabs;
                                }
                            }
                        }
                    }
                    tc_fence_before();
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_free[c]);
                }
            }
        }
    }

    if (warp >= 2 && (warp & 3) == 0 && lane == 0) tma_store_wait_all();  // this thread's output stores have landed
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, G::kTmemCols);
    }
}

}  // namespace fwd

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
static bool width_ok(int d) { return d == 16 || d == 32 || d == 64 || d == 128; }

bool tc_forward_supported(const MlpConfig& c)
{
    if (c.n_layers < 2 || c.n_layers > 5) return false;
    if (c.dtype != MLP_BF16 && c.dtype != MLP_F16) return false;
    if (c.input_dtype != c.dtype || c.encoding != MLP_ENC_NONE) return false;
    const int din = c.dims[0], dh = c.dims[1], dout = c.dims[c.n_layers];
    for (int l = 1; l < c.n_layers; ++l)
        if (c.dims[l] != dh) return false;
    if (!width_ok(din) || !width_ok(dh) || !width_ok(dout)) return false;
    // shapes that are instantiated below
    const bool constant_width = (din == dh && dh == dout && c.n_layers == 4);
    const bool wide = (din == 64 && dh == 128 && dout == 64 && c.n_layers == 5);
    if (!constant_width && !wide) return false;
    if (constant_width && !(c.hidden_act == MLP_ACT_RELU && c.output_act == MLP_ACT_IDENTITY)) return false;
    if (wide && !(c.hidden_act == MLP_ACT_GELU_TANH && c.output_act == MLP_ACT_IDENTITY)) return false;
    return true;
}

template <int DIN, int DH, int DOUT, int NL, int FMT, int ACT, int OUT_ACT, int NCH, int CS, int CPS = 1, int NCW = 1>
static cudaError_t launch_fwd(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const MlpForwardParams& a, std::string* err)
{
    using G = fwd::Geometry<DIN, DH, DOUT, NL, NCH, CS>;
    static_assert((G::kSmemBytes + (CPS > 1 ? 1024 : 0)) * CPS <= 227 * 1024, "shared memory budget");
    static_assert(G::kTmemCols * CPS <= 512, "tensor memory budget");
    CUtensorMap mx;
    const CUtensorMapDataType dt = FMT == MLP_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUtensorMapSwizzle sw = DIN >= 64 ? CU_TENSOR_MAP_SWIZZLE_128B : DIN == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    if (!make_tile_map(ws, &mx, dt, 2, a.inputs, a.count, DIN, fwd::panel_w(DIN), 128, sw, err)) return cudaErrorInvalidValue;
    if (a.outputs & 15u) { if (err) *err = "outputs must be 16-byte aligned"; return cudaErrorInvalidValue; }
    CUtensorMap mo;
    {
        constexpr int SC = G::kSlabCols;
        const CUtensorMapSwizzle so = SC == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : SC == 16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE;
        // with storage-type outputs the map is not used; describe the same memory as fp32 of half the width
        const uint32_t cols = (a.flags & MLP_FLAG_OUTPUT_STORAGE_TYPE) ? DOUT / 2 : DOUT;
        if (!make_tile_map(ws, &mo, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.outputs, a.count, cols, SC <= (int)cols ? SC : cols, 128, so, err))
            return cudaErrorInvalidValue;
    }
    fwd::Params p;
    p.net = (const MlpLayerPointers*)a.networkBuffer;
    p.out = (float*)a.outputs;
    p.status = ws->status;
    p.param_layout = c.param_layout;
    p.count = a.count;
    p.n_tiles = (a.count + 127u) / 128u;
    p.act_alpha = c.act_alpha;
    p.out_storage = (a.flags & MLP_FLAG_OUTPUT_STORAGE_TYPE) ? 1u : 0u;
    auto kern = fwd::forward_tc_kernel<DIN, DH, DOUT, NL, FMT, ACT, OUT_ACT, NCH, CS, CPS, NCW>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G::kSmemBytes);
    if (e != cudaSuccess) return e;
    const uint32_t slots = (uint32_t)ws->sm_count * (uint32_t)CPS;
    const uint32_t grid = p.n_tiles < slots ? p.n_tiles : slots;
    kern<<<grid, G::kThreads, G::kSmemBytes, st>>>(mx, mo, p);
    return cudaGetLastError();
}

cudaError_t launch_forward_tc(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const MlpForwardParams& a, int* launches,
                              std::string* err)
{
    if (!tc_forward_supported(c)) { if (err) *err = "shape not built for the tensor-core forward path"; return cudaErrorInvalidValue; }
    if (a.count == 0) return cudaSuccess;
    cudaError_t e = cudaErrorInvalidValue;
    const int w = c.dims[1];
    const bool wide = c.n_layers == 5;
    // chains per CTA, column split, CTAs per SM, control warps: the measured best per width
#define MLPB200_FWD(W_, FMT_, NCH_, CS_, CPS_, NCW_) \
    if (!wide && w == W_ && c.dtype == FMT_) e = launch_fwd<W_, W_, W_, 4, FMT_, MLP_ACT_RELU, MLP_ACT_IDENTITY, NCH_, CS_, CPS_, NCW_>(st, ws, c, a, err);
    MLPB200_FWD(16, MLP_F16, 2, 1, 3, 1) MLPB200_FWD(32, MLP_F16, 2, 1, 3, 1) MLPB200_FWD(64, MLP_F16, 6, 1, 1, 2) MLPB200_FWD(128, MLP_F16, 2, 2, 1, 1)
    MLPB200_FWD(16, MLP_BF16, 2, 1, 3, 1) MLPB200_FWD(32, MLP_BF16, 2, 1, 3, 1) MLPB200_FWD(64, MLP_BF16, 6, 1, 1, 2) MLPB200_FWD(128, MLP_BF16, 2, 2, 1, 1)
#undef MLPB200_FWD
    if (wide && c.dtype == MLP_BF16) e = launch_fwd<64, 128, 64, 5, MLP_BF16, MLP_ACT_GELU_TANH, MLP_ACT_IDENTITY, 2, 2>(st, ws, c, a, err);
    if (wide && c.dtype == MLP_F16) e = launch_fwd<64, 128, 64, 5, MLP_F16, MLP_ACT_GELU_TANH, MLP_ACT_IDENTITY, 2, 2>(st, ws, c, a, err);
    *launches += 1;
    return e;
}

}  // namespace mlpb200
