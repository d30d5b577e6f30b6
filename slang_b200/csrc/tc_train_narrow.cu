// learnGradient on the tensor cores for narrow networks: every layer width <= 64 (the fp16 CoopVec-style
// network 4-32-32-32-32-4 and the neural-texture network enc(2->32)-64-64-64-3).
//
// Every layer is padded to H x H in shared memory (zero rows and columns; H = 64, or 32 when every width
// fits), so one kernel shape serves all such networks: padded features stay exactly zero through the
// forward and backward pass.  Up to two tiles are in flight per CTA, each with its own operand buffers,
// working accumulator and epilogue warps.  (The shapes below are written for H = 64.)
// Orientation: the 128 samples of a tile run along the TMEM lanes (the MMA's M), features along the
// columns; an epilogue thread owns one sample row (or a column group of it).
//   forward   Z_l [128 x 64]  = A_l [128 x 64] . W_l^T        A: A_l, K-major          B: W_l [out][in], K-major
//   input     dA_l [128 x 64] = dZ_l [128 x 64] . W_l          A: dZ_l, K-major         B: W_l, MN-major
//   weights   dW_l | db_l [64 x 80] += dZ_l^T . [A_l | 1]      A: dZ_l, MN-major        B: A_l, then a tile whose first column
//             (one product of 64 rows, K = 128 samples)                                is ones, MN-major
// The thread that owns a sample builds the sample's input row itself (conversion or the frequency
// encoding), reads its targets straight from global memory, keeps the activation derivatives of its
// row in shared memory and keeps the running loss in registers.  Weight and bias gradients
// accumulate in tensor memory over all tiles of the CTA and leave through one atomic add per
// parameter per CTA.
//
// What the reference does instead: one thread per sample with per-element global atomics
// (examples/mlp-training/mlp_sw.slang:28-58) or CoopVec calls whose CPU/CUDA fallback is scalar loops
// (examples/mlp-training-coopvec/fflayer.slang:16-58, source/slang/hlsl.meta.slang:32835-32912).
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

namespace narrow {

using namespace layout;

constexpr int HMAX = 64;      // widest padded layer; the kernel is built for padded widths H = 64 and H = 32
constexpr int TS = 128;       // samples per tile
// Threads: warp 0 issues the products, warp 1 owns the tensor-memory allocation, then CS groups of four
// epilogue warps; group g handles columns [g * H / CS, (g + 1) * H / CS) of every row (H: the padded width).
constexpr int threads_for(int cs) { return 64 + 128 * cs; }

enum : uint32_t { kStatusCtrl = 0x1000u, kStatusEpi = 0x2000u };

struct Params {
    MlpConfig cfg;
    const MlpLayerPointers* net;
    uint32_t* loss_words;
    uint32_t* status;
    const void* inputs;
    const void* targets;
    float* input_grads;   // optional: [count][dims[0]] gradient with respect to the (unencoded) inputs
    float* outputs;       // optional: forward only; fp32 [count][dims[n_layers]] network outputs, nothing else is written
    uint32_t count;
    uint32_t n_tiles;
#ifdef MLPB200_TRACE
    unsigned long long* timing;   // developer builds only: time stamps of one round of CTA 0
#endif
};

// Developer builds (-DMLPB200_TRACE, never the shipped library) record clock64() stamps of the hand-offs of
// one round of CTA 0: control warp slot (step * NCH + chain) * 3 + {wait begins, wait ends, products issued},
// epilogue (first thread of each chain) slot 128 + (chain * 11 + step) * 2 + {woken, released}.
#ifdef MLPB200_TRACE
#define MLPB200_NTRACE(cond, slot) do { if (cond) p.timing[slot] = (unsigned long long)clock64(); } while (0)
constexpr uint32_t kTraceRound = 3;
#else
#define MLPB200_NTRACE(cond, slot) do { } while (0)
#endif

template <int FMT> struct Cvt;
template <> struct Cvt<MLP_BF16> {
    static constexpr uint32_t kUmmaFmt = 1;
    __device__ static __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi)
    {
        __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&t);
    }
    __device__ static __forceinline__ float lo(uint32_t p) { return __uint_as_float(p << 16); }
    __device__ static __forceinline__ float hi(uint32_t p) { return __uint_as_float(p & 0xffff0000u); }
    __device__ static __forceinline__ uint16_t one() { return 0x3F80; }
    // max(z, 0) of a pair; a zero z (either sign) comes out as a negative zero
    __device__ static __forceinline__ uint32_t relu_marked(uint32_t z2)
    {
        const __nv_bfloat162 z = *reinterpret_cast<const __nv_bfloat162*>(&z2), zero = __floats2bfloat162_rn(0.0f, 0.0f);
        const __nv_bfloat162 r = __hmax2(z, zero);
        return (*reinterpret_cast<const uint32_t*>(&r) & 0x7fff7fffu) | (__heq2_mask(z, zero) & 0x80008000u);
    }
    // 0xffff in the halves whose value is above zero
    __device__ static __forceinline__ uint32_t positive_mask(uint32_t a2)
    {
        return __hgt2_mask(*reinterpret_cast<const __nv_bfloat162*>(&a2), __floats2bfloat162_rn(0.0f, 0.0f));
    }
    // z < 0 ? round(alpha z) : z of a pair; the sign bit of the result is set exactly where z < 0
    __device__ static __forceinline__ uint32_t leaky_signed(uint32_t z2, float alpha)
    {
        const uint32_t m = __hlt2_mask(*reinterpret_cast<const __nv_bfloat162*>(&z2), __floats2bfloat162_rn(0.0f, 0.0f));
        return (pack2(__fmul_rn(alpha, lo(z2)), __fmul_rn(alpha, hi(z2))) & m) | (z2 & 0x7fff7fffu & ~m);
    }
};
template <> struct Cvt<MLP_F16> {
    static constexpr uint32_t kUmmaFmt = 0;
    __device__ static __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi)
    {
        __half2 t = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&t);
    }
    __device__ static __forceinline__ float lo(uint32_t p) { return __half2float(__ushort_as_half((uint16_t)(p & 0xffffu))); }
    __device__ static __forceinline__ float hi(uint32_t p) { return __half2float(__ushort_as_half((uint16_t)(p >> 16))); }
    __device__ static __forceinline__ uint16_t one() { return 0x3C00; }
    __device__ static __forceinline__ uint32_t relu_marked(uint32_t z2)
    {
        const __half2 z = *reinterpret_cast<const __half2*>(&z2), zero = __floats2half2_rn(0.0f, 0.0f);
        const __half2 r = __hmax2(z, zero);
        return (*reinterpret_cast<const uint32_t*>(&r) & 0x7fff7fffu) | (__heq2_mask(z, zero) & 0x80008000u);
    }
    __device__ static __forceinline__ uint32_t positive_mask(uint32_t a2)
    {
        return __hgt2_mask(*reinterpret_cast<const __half2*>(&a2), __floats2half2_rn(0.0f, 0.0f));
    }
    __device__ static __forceinline__ uint32_t leaky_signed(uint32_t z2, float alpha)
    {
        const uint32_t m = __hlt2_mask(*reinterpret_cast<const __half2*>(&z2), __floats2half2_rn(0.0f, 0.0f));
        return (pack2(__fmul_rn(alpha, lo(z2)), __fmul_rn(alpha, hi(z2))) & m) | (z2 & 0x7fff7fffu & ~m);
    }
};

// Shared-memory map for NL layers and NCH tiles in flight (bytes from a 1024-aligned base).  DFA: the
// activation derivative is read back from the stored activation instead of being kept in its own buffer.
template <int NL, int NCH, bool DFA, int H>
struct Map {
    static constexpr uint32_t kMat = H * H * 2;                // one padded weight matrix: H rows of 2 H bytes
    static constexpr uint32_t kTile = 128 * H * 2;             // one [128][H] operand tile
    static constexpr uint32_t kW = 0;                          // NL padded weight matrices
    static constexpr uint32_t kChain = kW + NL * kMat;         // per tile in flight:
    static constexpr uint32_t kA = 0;                          //   A_0 .. A_{NL-1}: layer inputs; dZ_{l-1} later replaces A_l
    static constexpr uint32_t kD = kA + NL * kTile;            //   activation derivatives of layers 0 .. NL-2 (absent with DFA)
    static constexpr uint32_t kDZ = kD + (DFA ? 0 : (NL - 1) * kTile);   //   dZ of the last layer
    static constexpr uint32_t kChainBytes = kDZ + kTile;
    // The ones tile (first column one, rest zero): [128 rows][H elements] in the layout of an activation tile, so
    // that its first 16 columns can follow A_l as a further block of the weight-gradient product's B operand:
    // dW_l | db_l come out of one product of N = H + 16, H + 16 accumulator columns per layer.
    static constexpr uint32_t kOnes = kChain + NCH * kChainBytes;
    static constexpr uint32_t kBias = kOnes + kTile;        // fp32 [NL][H]
    static constexpr uint32_t kBars = kBias + NL * H * 4;      // per chain: acc_full, acc_free, tile_done
    static constexpr uint32_t kTmemPtr = kBars + 3 * NCH * 8;
    static constexpr uint32_t kAbort = kTmemPtr + 4;
    static constexpr uint32_t kSmemBytes = kAbort + 4 + 1024;
    // tensor-memory columns: one working accumulator per chain, then the gradients (shared by the chains)
    static constexpr uint32_t kColAcc = 0, kColDW = H * NCH, kDwCols = H + 16;  // columns per layer: dW_l, then db_l
    static constexpr uint32_t kTmemCols = 512;
    static_assert(kColDW + kDwCols * NL <= 512, "tensor memory budget");
    // tensor-memory column of layer l's bias gradient
    __host__ __device__ static constexpr uint32_t col_db(int l) { return kColDW + kDwCols * l + H; }
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

// HACT / OACT: the hidden and output activation as compile-time constants, or -1 to read them from
// the configuration at run time (slower: every element goes through a switch).
// CS: column split of the epilogue (1, 2 or 4 groups of four warps).  The loss of a sample is summed by
// the group that holds the output columns, so CS > 1 needs the output width to fit one group (64 / CS).
// NCH: tiles in flight per CTA ("chains"): each has its own operand buffers, working accumulator,
// barriers and epilogue warps, and both accumulate into the same gradient columns; while one chain's
// epilogue runs, the tensor pipe works on the other chain's product.
// DFA: derivative-from-activation form (ReLU only), which frees the derivative buffers: the forward
// epilogue stores max(z, 0) and marks z == 0 with a negative zero, so the backward epilogue recovers
// the derivative 1 / one half / 0 exactly from the stored value (a negative zero is a zero to every
// product that reads the buffer).
// H: the padded width of every layer, 64 (128-byte operand rows, 128-byte swizzle) or 32 (64-byte rows,
// 64-byte swizzle; a quarter of the shared memory and half of the epilogue work per tile).
template <int NL, int FMT, int HACT, int OACT, int CS, int NCH, bool DFA, int H>
__global__ void __launch_bounds__(threads_for(CS * NCH), 1) learn_gradient_narrow_kernel(const Params p)
{
    constexpr int kThreads = threads_for(CS * NCH);
    constexpr int GW = H / CS;   // columns per epilogue group
    static_assert(H == 64 || H == 32, "padded width");
    static_assert(GW % 16 == 0, "an epilogue group works on whole 16-column accumulator reads");
    static_assert(!DFA || HACT == MLP_ACT_RELU || HACT == MLP_ACT_LEAKY_RELU,
                  "the derivative is recovered from the activation only for ReLU and leaky ReLU");
    using M = Map<NL, NCH, DFA, H>;
    using C = Cvt<FMT>;
    constexpr uint32_t kMat = M::kMat, kTile = M::kTile;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    uint64_t* bars = (uint64_t*)(smem + M::kBars);   // [chain][acc_full, acc_free, tile_done]
    uint32_t* tmem_ptr = (uint32_t*)(smem + M::kTmemPtr);
    volatile uint32_t* abort_flag = (volatile uint32_t*)(smem + M::kAbort);
    float* s_bias = (float*)(smem + M::kBias);
    const MlpConfig& c = p.cfg;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n_my_tiles = (p.n_tiles > blockIdx.x) ? (p.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (threadIdx.x == 0) {
        for (int h = 0; h < NCH; ++h) {
            mbar_init(&bars[3 * h + 0], 1);
            mbar_init(&bars[3 * h + 1], 4 * CS);
            mbar_init(&bars[3 * h + 2], 1);
        }
        *abort_flag = 0u;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_ptr, M::kTmemCols);
        tmem_relinquish();
    }
    // Padded weights (zero outside [out][in]), biases, and the ones column.
    for (int l = 0; l < NL; ++l) {
        const int in = c.dims[l], out = c.dims[l + 1];
        // 16-bit storage: the stored bits; fp32 storage with 16-bit operands (MlpConfig.operand_dtype): converted here
        const uint16_t* W = (const uint16_t*)p.net[l].weights;
        const float* W32 = (const float*)p.net[l].weights;
        for (int idx = threadIdx.x; idx < H * H; idx += kThreads) {
            const int o = idx / H, i = idx % H;
            uint16_t v = 0;
            if (o < out && i < in) {
                const int64_t wi = weight_index(c.param_layout, in, out, o, i);
                v = c.dtype == MLP_F32 ? (uint16_t)(C::pack2(W32[wi], 0.0f) & 0xffffu) : W[wi];
            }
            *(uint16_t*)(smem + M::kW + l * kMat + chunk_offset<H>(H, o, i / 8) + (i % 8) * 2) = v;
        }
        for (int j = threadIdx.x; j < H; j += kThreads)
            s_bias[l * H + j] = j < out ? load_as_f32(c.dtype, (const void*)p.net[l].biases, j) : 0.0f;
    }
    for (int idx = threadIdx.x; idx < 128 * H; idx += kThreads) {
        const int r = idx / H, i = idx % H;
        *(uint16_t*)(smem + M::kOnes + chunk_offset<H>(128, r, i / 8) + (i % 8) * 2) = (i == 0) ? C::one() : (uint16_t)0;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    if (warp == 0) {
        // =================================== control warp ==========================================
        // Chain h works on this CTA's tiles h, h + NCH, h + 2 NCH, ...; the warp walks the layer schedule
        // once per round and serves the chains in turn at every step.
        if (n_my_tiles > 0) {
            const bool leader = elect_one();
            constexpr uint32_t F = C::kUmmaFmt;
            constexpr uint32_t kIdFwd = umma_idesc(F, 0, 0, 128, H);   // acts (K) x W (K)
            constexpr uint32_t kIdDx = umma_idesc(F, 0, 1, 128, H);    // dZ (K) x W (MN)
            const uint32_t lo_base = (sbase & 0x3FFFFu) >> 4;
            // operand rows of 2 H bytes with the swizzle of that span; groups of eight rows are 16 H bytes apart
            constexpr uint32_t kRow = (uint32_t)row_bytes(H);
            constexpr uint32_t kHi128 = ((8u * kRow) >> 4) | (1u << 14) | (layout_type(H) << 29);
            // K-major [rows][H]: a K step of 16 elements is 32 bytes inside the row.
            auto desc_k = [&](uint32_t buf, int k) -> uint64_t {
                return ((uint64_t)kHi128 << 32) | (lo_base + ((buf + (uint32_t)k * 32u) >> 4) + (1u << 16));
            };
            // MN-major [K rows][H]: a K step is 16 rows; a further H-element block, where the instruction
            // asks for 128 rows of output, starts 16 bytes further (its results are never read).
            auto desc_mn = [&](uint32_t buf, int k) -> uint64_t {
                return ((uint64_t)kHi128 << 32) | (lo_base + ((buf + (uint32_t)k * 16u * kRow) >> 4) + (1u << 16));
            };
            // The same with the second H-element block `lbo` bytes after the first (the B operand [A_l | ones]).
            auto desc_mn_lbo = [&](uint32_t buf, int k, uint32_t lbo) -> uint64_t {
                return ((uint64_t)kHi128 << 32) | (lo_base + ((buf + (uint32_t)k * 16u * kRow) >> 4) + ((lbo >> 4) << 16));
            };
            constexpr uint32_t kIdDwDb = umma_idesc(F, 1, 1, 64, H + 16);    // dZ^T (MN, 64 rows) x [acts | ones] (MN)
            uint32_t n_free[NCH];  // acc_free phases observed, per chain
#pragma unroll
            for (int h = 0; h < NCH; ++h) n_free[h] = 0;
            bool ok = true;
#ifdef MLPB200_TRACE
            bool tr_on = false;
            int tr_step = 0;
#endif
            auto wait_free = [&](int h) {
                MLPB200_NTRACE(tr_on, (tr_step * NCH + h) * 3 + 0);
                ok = ok && mbar_wait(&bars[3 * h + 1], n_free[h] & 1u, abort_flag, p.status, kStatusCtrl);
                ++n_free[h];
                tc_fence_after();
                MLPB200_NTRACE(tr_on, (tr_step * NCH + h) * 3 + 1);
            };
            // dW_l and db_l of a tile; `first` is true only for the launch's first product into them.
            auto grads = [&](int l, uint32_t dzbuf, uint32_t abuf, bool first) {
#pragma unroll
                for (int k = 0; k < TS / 16; ++k)
                    umma_f16(tmem_base + M::kColDW + (uint32_t)l * M::kDwCols, desc_mn(dzbuf, k), desc_mn_lbo(abuf, k, M::kOnes - abuf),
                             kIdDwDb, (first && k == 0) ? 0u : 1u);
            };
            const uint32_t rounds = (n_my_tiles + NCH - 1) / NCH;
            for (uint32_t rd = 0; rd < rounds && ok; ++rd) {
#ifdef MLPB200_TRACE
                tr_on = leader && blockIdx.x == 0 && rd == kTraceRound && p.timing;
#endif
                // ---- forward ----
#pragma unroll
                for (int l = 0; l < NL; ++l) {
#ifdef MLPB200_TRACE
                    tr_step = l;
#endif
#pragma unroll
                    for (int h = 0; h < NCH; ++h) {
                        if (rd * NCH + h >= n_my_tiles) continue;
                        const uint32_t cb = M::kChain + (uint32_t)h * M::kChainBytes;
                        wait_free(h);  // A_l is in shared memory (l = 0: the input rows) and the accumulator is drained
                        if (ok) {
                            if (leader) {
#pragma unroll
                                for (int k = 0; k < H / 16; ++k)
                                    umma_f16(tmem_base + M::kColAcc + (uint32_t)(h * H), desc_k(cb + M::kA + (uint32_t)l * kTile, k),
                                             desc_k(M::kW + (uint32_t)l * kMat, k), kIdFwd, k > 0);
                                umma_commit(&bars[3 * h + 0]);
                                MLPB200_NTRACE(tr_on, (tr_step * NCH + h) * 3 + 2);
                            }
                            __syncwarp();
                        }
                    }
                }
                if (p.outputs) continue;   // forward only: the next round's layer 0 waits for the epilogue as usual
                // ---- backward ----
#pragma unroll
                for (int l = NL - 1; l >= 1; --l) {
#ifdef MLPB200_TRACE
                    tr_step = NL + (NL - 1 - l);
#endif
#pragma unroll
                    for (int h = 0; h < NCH; ++h) {
                        if (rd * NCH + h >= n_my_tiles) continue;
                        const uint32_t cb = M::kChain + (uint32_t)h * M::kChainBytes;
                        wait_free(h);  // dZ_l is in shared memory
                        if (ok) {
                            const uint32_t dzbuf = cb + ((l == NL - 1) ? M::kDZ : M::kA + (uint32_t)(l + 1) * kTile);
                            if (leader) {
#pragma unroll
                                for (int k = 0; k < H / 16; ++k)
                                    umma_f16(tmem_base + M::kColAcc + (uint32_t)(h * H), desc_k(dzbuf, k), desc_mn(M::kW + (uint32_t)l * kMat, k),
                                             kIdDx, k > 0);
                                grads(l, dzbuf, cb + M::kA + (uint32_t)l * kTile, rd == 0 && h == 0);
                                umma_commit(&bars[3 * h + 0]);
                                MLPB200_NTRACE(tr_on, (tr_step * NCH + h) * 3 + 2);
                            }
                            __syncwarp();
                        }
                    }
                }
#ifdef MLPB200_TRACE
                tr_step = 2 * NL - 1;
#endif
#pragma unroll
                for (int h = 0; h < NCH; ++h) {
                    if (rd * NCH + h >= n_my_tiles) continue;
                    const uint32_t cb = M::kChain + (uint32_t)h * M::kChainBytes;
                    wait_free(h);  // dZ_0 is in shared memory (in A_1's buffer, or the last layer's own buffer)
                    if (ok) {
                        const uint32_t dz0 = cb + (NL == 1 ? M::kDZ : M::kA + kTile);
                        if (leader) {
                            if (p.input_grads) {
                                // the input gradient dA_0 = dZ_0 . W_0, wanted by an encoder in front of the network
#pragma unroll
                                for (int k = 0; k < H / 16; ++k)
                                    umma_f16(tmem_base + M::kColAcc + (uint32_t)(h * H), desc_k(dz0, k), desc_mn(M::kW, k), kIdDx, k > 0);
                            }
                            grads(0, dz0, cb + M::kA, rd == 0 && h == 0);
                            if (p.input_grads) umma_commit(&bars[3 * h + 0]);
                            umma_commit(&bars[3 * h + 2]);
                            MLPB200_NTRACE(tr_on, (tr_step * NCH + h) * 3 + 2);
                        }
                        __syncwarp();
                        if (p.input_grads) wait_free(h);  // the epilogue has read dA_0 out of the accumulator
                    }
                }
            }
        }
    } else if (warp >= 2) {
        // =================================== epilogue warps ========================================
        const int q = warp & 3;       // a warp reaches the 32 tensor-memory lanes of its index modulo four
        const int r = q * 32 + lane;  // the sample row (TMEM lane) this thread works on
        const int h = (warp - 2) / (4 * CS);          // the chain (tile in flight) this warp serves
        const int g = ((warp - 2) >> 2) % CS;
        const int cbeg = g * GW, cend = cbeg + GW;   // this thread's columns of the row
        uint64_t* acc_full = &bars[3 * h + 0];
        uint64_t* acc_free = &bars[3 * h + 1];
        uint64_t* tile_done = &bars[3 * h + 2];
        const uint32_t cb = M::kChain + (uint32_t)h * M::kChainBytes;
        const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + M::kColAcc + (uint32_t)(h * H);
        const int od = c.dims[NL];
        const int hact = HACT >= 0 ? HACT : c.hidden_act;
        const int oact = OACT >= 0 ? OACT : c.output_act;
        const float loss_scale = c.loss == MLP_LOSS_MSE_MEAN ? 1.0f / (float)od : 1.0f;
        float run_max = 0.0f, run_sum = 0.0f;
        uint32_t n_full = 0;
        bool ok = true;
        // Pre-activations, outputs and input gradients are rounded to the storage type; with fp32 storage (16-bit
        // operands only) they stay as they are.
        const bool fp32_storage = c.dtype == MLP_F32;
        auto round_z = [&](float v) -> float { return fp32_storage ? v : C::round(v); };
        const float alpha_op = C::round(c.act_alpha);
        // few outputs (they sit in column group 0): their targets are read at the start of the tile
        const bool t_pre = !p.outputs && od <= 4 && g == 0;
        float tpre[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#ifdef MLPB200_TRACE
        bool tr_on = false;
        int tr_step = 0;
#endif
        auto release = [&]() {
            tc_fence_before();
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_free);
            MLPB200_NTRACE(tr_on, 128 + (h * 11 + tr_step) * 2 + 1);
#ifdef MLPB200_TRACE
            ++tr_step;
#endif
        };
        auto wait_full = [&]() {
            ok = ok && mbar_wait(acc_full, n_full & 1u, abort_flag, p.status, kStatusEpi);
            ++n_full;
            tc_fence_after();
            MLPB200_NTRACE(tr_on, 128 + (h * 11 + tr_step) * 2 + 0);
        };
        auto row_chunk = [&](uint32_t buf, int j) -> uint4* { return (uint4*)(smem + cb + buf + chunk_offset<H>(128, r, j)); };
        const uint32_t n_chain_tiles = n_my_tiles > (uint32_t)h ? (n_my_tiles - (uint32_t)h + NCH - 1) / NCH : 0;

        for (uint32_t it = 0; it < n_chain_tiles && ok; ++it) {
            const uint64_t tile = (uint64_t)blockIdx.x + ((uint64_t)it * NCH + (uint64_t)h) * gridDim.x;
            const uint64_t sample = tile * TS + (uint64_t)r;
            const bool valid = sample < p.count;
#ifdef MLPB200_TRACE
            tr_on = blockIdx.x == 0 && it == kTraceRound && p.timing && r == 0 && g == 0;
            tr_step = 0;
            MLPB200_NTRACE(tr_on, 128 + (h * 11) * 2 + 0);
#endif
            // ---- the input row: conversion (and zero padding) or the frequency encoding ----
            // training: dW_0 of the chain's previous tile still reads A_0 until tile_done, so the row is stored
            // after that wait; forward only: the layer-0 product that read it has long completed (its
            // accumulator was consumed)
            {
                // Blocks of 16 columns are dealt to the column groups in turn, so the groups share the real input
                // columns (and the two coordinates of the frequency encoding) whatever the padding.  The row is
                // built in registers first: the loads and the sines overlap the wait below.
                constexpr int kBlocks = GW / 16;
                uint4 xa[kBlocks], xb[kBlocks];
                // up to four targets per sample are fetched here too, a whole forward pass ahead of their use
                if (t_pre && valid) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (i < od) tpre[i] = load_as_f32(c.target_dtype, p.targets, sample * od + i);
                }
#pragma unroll
                for (int b = 0; b < kBlocks; ++b) {
                    const int c0 = 16 * (g + CS * b);
                    float x[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) x[i] = 0.0f;
                    if (valid) {
                        if (c.encoding == MLP_ENC_FREQ2D) {
                            // features [16u, 16u + 16) are sin/cos of 2^k pi times coordinate u, k = 0..7
                            if (c0 < 32) {
                                const float v = load_as_f32(c.input_dtype, p.inputs, sample * 2 + (c0 >> 4));
#pragma unroll
                                for (int k = 0; k < 8; ++k) {
                                    const float arg = ldexpf(3.14159265358979323846f, k) * v;
                                    sincosf(arg, &x[k * 2 + 0], &x[k * 2 + 1]);
                                }
                            }
                        } else if (c0 < c.dims[0]) {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (c0 + i < c.dims[0]) x[i] = load_as_f32(c.input_dtype, p.inputs, sample * c.dims[0] + c0 + i);
                        }
                    }
                    xa[b] = make_uint4(C::pack2(x[0], x[1]), C::pack2(x[2], x[3]), C::pack2(x[4], x[5]), C::pack2(x[6], x[7]));
                    xb[b] = make_uint4(C::pack2(x[8], x[9]), C::pack2(x[10], x[11]), C::pack2(x[12], x[13]), C::pack2(x[14], x[15]));
                }
                if (it > 0 && !p.outputs) ok = ok && mbar_wait(tile_done, (it - 1) & 1u, abort_flag, p.status, kStatusEpi);
                if (!ok) break;
#pragma unroll
                for (int b = 0; b < kBlocks; ++b) {
                    const int c0 = 16 * (g + CS * b);
                    *row_chunk(M::kA, c0 / 8) = xa[b];
                    *row_chunk(M::kA, c0 / 8 + 1) = xb[b];
                }
                release();
            }
            // ---- forward ----
#pragma unroll
            for (int l = 0; l < NL; ++l) {
                wait_full();
                if (ok) {
                    const bool last = (l == NL - 1);
                    float loss = 0.0f;
                    const int width = c.dims[l + 1];  // real features of this layer; the padding beyond stays zero
                    if (last && p.outputs) {
                        // forward only: the output activation of the real columns goes to global memory.  No
                        // separate release: the release after the next tile's input row (same warps, program
                        // order) tells the control warp that this accumulator is drained.
#pragma unroll
                        for (int c0 = cbeg; c0 < cend; c0 += 16) {
                            if (c0 >= width) continue;
                            uint32_t v[16];
                            tmem_ld_32x16(t_acc + (uint32_t)c0, v);
                            tmem_ld_wait();
                            if (valid) {
                                float* dst = p.outputs + sample * (uint64_t)od + c0;
#pragma unroll
                                for (int i = 0; i < 16; ++i)
                                    if (c0 + i < od)
                                        dst[i] = act_value(oact, c.act_alpha, round_z(__uint_as_float(v[i]) + s_bias[l * H + c0 + i]));
                            }
                        }
                        tc_fence_before();
                        continue;
                    }
#pragma unroll
                    for (int c0 = cbeg; c0 < cend; c0 += 16) {
                        const uint32_t abuf = last ? M::kDZ : M::kA + (uint32_t)(l + 1) * kTile;
                        if (c0 >= width) {
                            *row_chunk(abuf, c0 / 8) = make_uint4(0u, 0u, 0u, 0u);
                            *row_chunk(abuf, c0 / 8 + 1) = make_uint4(0u, 0u, 0u, 0u);
                            continue;
                        }
                        uint32_t v[16];
                        tmem_ld_32x16(t_acc + (uint32_t)c0, v);
                        tmem_ld_wait();
                        uint32_t pa[8], pd[8];
                        if constexpr (DFA) {
                            if (!last && !fp32_storage) {
                                // ReLU and leaky ReLU on pairs: bias, one paired rounding of the pre-activations,
                                // the activation on the packed pair with the derivative's case kept in the sign bit
#pragma unroll
                                for (int k = 0; k < 16; k += 4) {
                                    const float4 b4 = *(const float4*)(s_bias + l * H + c0 + k);
                                    const uint32_t z01 = C::pack2(__uint_as_float(v[k]) + b4.x, __uint_as_float(v[k + 1]) + b4.y);
                                    const uint32_t z23 = C::pack2(__uint_as_float(v[k + 2]) + b4.z, __uint_as_float(v[k + 3]) + b4.w);
                                    if constexpr (HACT == MLP_ACT_RELU) {
                                        pa[k >> 1] = C::relu_marked(z01);
                                        pa[(k >> 1) + 1] = C::relu_marked(z23);
                                    } else {
                                        pa[k >> 1] = C::leaky_signed(z01, c.act_alpha);
                                        pa[(k >> 1) + 1] = C::leaky_signed(z23, c.act_alpha);
                                    }
                                }
                                *row_chunk(abuf, c0 / 8) = make_uint4(pa[0], pa[1], pa[2], pa[3]);
                                *row_chunk(abuf, c0 / 8 + 1) = make_uint4(pa[4], pa[5], pa[6], pa[7]);
                                continue;
                            }
                        }
#pragma unroll
                        for (int k = 0; k < 16; k += 4) {
                            const float4 b4 = *(const float4*)(s_bias + l * H + c0 + k);
                            const float bb[4] = {b4.x, b4.y, b4.z, b4.w};
                            float a4[4], d4[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int j = c0 + k + e;
                                const float z = round_z(__uint_as_float(v[k + e]) + bb[e]);
                                if (!last) {
                                    if constexpr (DFA && HACT == MLP_ACT_RELU) {
                                        // max(z, 0), with z == 0 stored as a negative zero: the backward epilogue
                                        // tells "below zero", "zero" and "above zero" apart by the stored bits
                                        a4[e] = z > 0.0f ? z : (z == 0.0f ? -0.0f : 0.0f);
                                        d4[e] = 0.0f;
                                    } else if constexpr (DFA) {
                                        // leaky ReLU: the sign bit of the stored value is "z < 0" (alpha z keeps its
                                        // sign when it rounds to zero; a zero z is stored as a positive zero)
                                        a4[e] = z < 0.0f ? __fmul_rn(c.act_alpha, z) : (z == 0.0f ? 0.0f : z);
                                        d4[e] = 0.0f;
                                    } else {
                                        a4[e] = act_value(hact, c.act_alpha, z);
                                        d4[e] = act_deriv(hact, c.act_alpha, z);
                                    }
                                } else {
                                    // loss and dZ of the last layer; padded outputs and rows past the batch give zero
                                    float dz = 0.0f;
                                    if (valid && j < od) {
                                        const float o = act_value(oact, c.act_alpha, z);
                                        const float diff = o - (t_pre ? tpre[(k + e) & 3] : load_as_f32(c.target_dtype, p.targets, sample * od + j));
                                        loss = fmaf(diff * loss_scale, diff, loss);
                                        dz = ((2.0f * loss_scale) * diff) * act_deriv(oact, c.act_alpha, z);
                                    }
                                    a4[e] = dz;
                                    d4[e] = 0.0f;
                                }
                            }
                            pa[k >> 1] = C::pack2(a4[0], a4[1]);
                            pa[(k >> 1) + 1] = C::pack2(a4[2], a4[3]);
                            pd[k >> 1] = C::pack2(d4[0], d4[1]);
                            pd[(k >> 1) + 1] = C::pack2(d4[2], d4[3]);
                        }
                        *row_chunk(abuf, c0 / 8) = make_uint4(pa[0], pa[1], pa[2], pa[3]);
                        *row_chunk(abuf, c0 / 8 + 1) = make_uint4(pa[4], pa[5], pa[6], pa[7]);
                        if constexpr (!DFA) {
                            if (!last && !p.outputs) {
                                *row_chunk(M::kD + (uint32_t)l * kTile, c0 / 8) = make_uint4(pd[0], pd[1], pd[2], pd[3]);
                                *row_chunk(M::kD + (uint32_t)l * kTile, c0 / 8 + 1) = make_uint4(pd[4], pd[5], pd[6], pd[7]);
                            }
                        }
                    }
                    if (last) {
                        run_max = fmaxf(run_max, loss);
                        run_sum += loss;
                    }
                    release();
                }
            }
            if (p.outputs) continue;   // forward only
            // the chain's next tile: start its input and target rows on their way into the L2 cache
            if (g == 0 && it + 1 < n_chain_tiles) {
                const uint64_t ns = sample + (uint64_t)NCH * gridDim.x * TS;
                if (ns < p.count) {
                    const uint64_t in_w = c.encoding == MLP_ENC_FREQ2D ? 2u : (uint64_t)c.dims[0];
                    const char* xi = (const char*)p.inputs + ns * in_w * (c.input_dtype == MLP_F32 ? 4u : 2u);
                    const char* ti = (const char*)p.targets + ns * (uint64_t)od * (c.target_dtype == MLP_F32 ? 4u : 2u);
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(xi));
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(ti));
                }
            }
            // ---- backward: dA_l in the accumulator times the derivative gives dZ_{l-1}, written over A_l ----
#pragma unroll
            for (int l = NL - 1; l >= 1; --l) {
                wait_full();
                if (ok) {
                    const int width = c.dims[l];  // real features of dZ_{l-1}
#pragma unroll
                    for (int c0 = cbeg; c0 < cend; c0 += 16) {
                        if (c0 >= width) {
                            *row_chunk(M::kA + (uint32_t)l * kTile, c0 / 8) = make_uint4(0u, 0u, 0u, 0u);
                            *row_chunk(M::kA + (uint32_t)l * kTile, c0 / 8 + 1) = make_uint4(0u, 0u, 0u, 0u);
                            continue;
                        }
                        uint32_t v[16];
                        tmem_ld_32x16(t_acc + (uint32_t)c0, v);
                        tmem_ld_wait();
                        const uint32_t dbuf = DFA ? M::kA + (uint32_t)l * kTile : M::kD + (uint32_t)(l - 1) * kTile;
                        const uint4 d0 = *row_chunk(dbuf, c0 / 8);
                        const uint4 d1 = *row_chunk(dbuf, c0 / 8 + 1);
                        const uint32_t dd[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
                        uint32_t pz[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            if constexpr (DFA && HACT == MLP_ACT_RELU) {
                                // no "z was exactly zero" mark in the pair: the rounded dA where the activation is
                                // positive, zero elsewhere
                                if ((dd[k] & 0x80008000u) == 0u) {
                                    pz[k] = C::pack2(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1])) & C::positive_mask(dd[k]);
                                    continue;
                                }
                            }
                            if constexpr (DFA && HACT == MLP_ACT_LEAKY_RELU) {
                                // alpha dA where the stored sign says z < 0, dA elsewhere, each rounded once
                                const float g0 = __uint_as_float(v[2 * k]), g1 = __uint_as_float(v[2 * k + 1]);
                                const uint32_t m = ((dd[k] >> 15) & 0x00010001u) * 0xffffu;
                                pz[k] = (C::pack2(g0 * alpha_op, g1 * alpha_op) & m) | (C::pack2(g0, g1) & ~m);
                                continue;
                            }
                            float dl, dh;
                            if constexpr (DFA && HACT == MLP_ACT_RELU) {
                                // stored activation: positive -> 1, negative zero -> one half (z was 0), zero -> 0
                                const uint32_t lo16 = dd[k] & 0xffffu, hi16 = dd[k] >> 16;
                                dl = (lo16 & 0x7fffu) ? 1.0f : (lo16 ? 0.5f : 0.0f);
                                dh = (hi16 & 0x7fffu) ? 1.0f : (hi16 ? 0.5f : 0.0f);
                            } else if constexpr (DFA) {
                                // leaky ReLU: sign bit set -> alpha (rounded to the operand type like a stored derivative)
                                dl = (dd[k] & 0x8000u) ? alpha_op : 1.0f;
                                dh = (dd[k] & 0x80000000u) ? alpha_op : 1.0f;
                            } else {
                                dl = C::lo(dd[k]);
                                dh = C::hi(dd[k]);
                            }
                            pz[k] = C::pack2(__uint_as_float(v[2 * k]) * dl, __uint_as_float(v[2 * k + 1]) * dh);
                        }
                        *row_chunk(M::kA + (uint32_t)l * kTile, c0 / 8) = make_uint4(pz[0], pz[1], pz[2], pz[3]);
                        *row_chunk(M::kA + (uint32_t)l * kTile, c0 / 8 + 1) = make_uint4(pz[4], pz[5], pz[6], pz[7]);
                    }
                    release();
                }
            }
            // ---- optional: the input gradient rows, rounded to the storage type ----
            if (p.input_grads) {
                wait_full();
                if (ok) {
                    const int in0 = c.dims[0];
#pragma unroll
                    for (int c0 = cbeg; c0 < cend; c0 += 16) {
                        if (c0 >= in0) continue;
                        uint32_t v[16];
                        tmem_ld_32x16(t_acc + (uint32_t)c0, v);
                        tmem_ld_wait();
                        if (valid) {
                            float* dst = p.input_grads + sample * (uint64_t)in0 + c0;
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (c0 + i < in0) dst[i] = round_z(__uint_as_float(v[i]));
                        }
                    }
                    release();
                }
            }
        }

        // ---- one add per parameter per CTA: lane = output feature, column = input feature ----
        if (ok && n_chain_tiles > 0 && !p.outputs) ok = mbar_wait(tile_done, (n_chain_tiles - 1) & 1u, abort_flag, p.status, kStatusEpi);
        // Every epilogue warp arrives here, whatever happened before: after this barrier the last product
        // of every chain has completed (or the CTA is aborting).
        asm volatile("bar.sync 1, %0;" ::"n"(128 * CS * NCH) : "memory");
        if (ok && !*abort_flag && n_my_tiles > 0 && !p.outputs) {
            tc_fence_after();
            const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
            // the warp groups of all chains share the columns: group i takes the 16-column pieces i, i + G, ...
            constexpr int G = CS * NCH;
            // The gradient products have 64 rows: row r of such an accumulator sits on lane 32 (r / 16) + r % 16,
            // so the first 16 lanes of this warp's quarter hold the output features 16 q .. 16 q + 15.
            const int fo = q * 16 + lane;
            const bool has_row = lane < 16;
            for (int l = 0; l < NL; ++l) {
                const int in = c.dims[l], out = c.dims[l + 1];
                float* dW = (float*)p.net[l].weightsGrad;
                float* dB = (float*)p.net[l].biasesGrad;
                for (int c0 = (h * CS + g) * 16; c0 < H; c0 += 16 * G) {
                    uint32_t v[16];
                    tmem_ld_32x16(lane_base + M::kColDW + (uint32_t)l * M::kDwCols + (uint32_t)c0, v);
                    tmem_ld_wait();
                    if (has_row && fo < out) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (c0 + i < in) atomicAdd(dW + weight_index(c.param_layout, in, out, fo, c0 + i), __uint_as_float(v[i]));
                    }
                }
                if (h == 0 && g == 0) {
                    uint32_t b[16];
                    tmem_ld_32x16(lane_base + M::col_db(l), b);
                    tmem_ld_wait();
                    if (has_row && fo < out) atomicAdd(dB + fo, __uint_as_float(b[0]));
                }
            }
            float mx = run_max, sm = run_sum;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                sm += __shfl_xor_sync(0xffffffffu, sm, o);
            }
            if (lane == 0 && g == 0) {   // the output columns, and with them the loss, live in group 0 of each chain
                atomicMax(p.loss_words, __float_as_uint(mx));
                atomicAdd((float*)(p.loss_words + 1), sm);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, M::kTmemCols);
    }
}

}  // namespace narrow

#if MLPB200_NARROW_PART == 0
bool tc_train_narrow_supported(const MlpConfig& c)
{
    if (c.n_layers < 2 || c.n_layers > 5) return false;
    const int op = c.operand_dtype ? c.operand_dtype : c.dtype;  // fp32 storage runs here with 16-bit operands
    if (op != MLP_BF16 && op != MLP_F16) return false;
    for (int l = 0; l <= c.n_layers; ++l)
        if (c.dims[l] > narrow::HMAX) return false;
    if (c.encoding == MLP_ENC_FREQ2D && c.dims[0] != 32) return false;
    return true;
}
#endif

template <int NL, int FMT, int HACT, int OACT, int CS, int NCH = 1, bool DFA = false, int H = narrow::HMAX>
static cudaError_t launch_narrow_cs(cudaStream_t st, TcWorkspace* ws, const narrow::Params& p)
{
    using M = narrow::Map<NL, NCH, DFA, H>;
    auto kern = narrow::learn_gradient_narrow_kernel<NL, FMT, HACT, OACT, CS, NCH, DFA, H>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)M::kSmemBytes);
    if (e != cudaSuccess) return e;
    const uint32_t grid = p.n_tiles < (uint32_t)ws->sm_count ? p.n_tiles : (uint32_t)ws->sm_count;
#ifdef MLPB200_TRACE
    narrow::Params q = p;
    q.timing = ws->timing;
    kern<<<grid, narrow::threads_for(CS * NCH), M::kSmemBytes, st>>>(q);
#else
    kern<<<grid, narrow::threads_for(CS * NCH), M::kSmemBytes, st>>>(p);
#endif
    return cudaGetLastError();
}

// The widest column split whose group still holds every output column.
template <int NL, int FMT, int HACT, int OACT>
static cudaError_t launch_narrow(cudaStream_t st, TcWorkspace* ws, const narrow::Params& p)
{
    const int od = p.cfg.dims[NL];
    if (od <= narrow::HMAX / 4) return launch_narrow_cs<NL, FMT, HACT, OACT, 4>(st, ws, p);
    if (od <= narrow::HMAX / 2) return launch_narrow_cs<NL, FMT, HACT, OACT, 2>(st, ws, p);
    return launch_narrow_cs<NL, FMT, HACT, OACT, 1>(st, ws, p);
}

// The kernel is instantiated some fifty times (layer counts, formats, column splits, tiles in flight).
// This file is compiled once per MLPB200_NARROW_PART (0..7) so that the instantiations build side by
// side: part 0 holds the host entry points and the dispatcher, every part holds one group of builds.
#ifndef MLPB200_NARROW_PART
#error "compile with -DMLPB200_NARROW_PART=0..7 (slang_b200/build.py does)"
#endif

cudaError_t launch_narrow_fits32(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p);
cudaError_t launch_narrow_named(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p);
cudaError_t launch_narrow_relu2(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p);

#if MLPB200_NARROW_PART == 1
// Networks whose every width fits 32 (and whose outputs fit one 16-column epilogue group) run the
// 32-wide build: operand tiles a quarter of the size, so two tiles are in flight with every buffer kept.
cudaError_t launch_narrow_fits32(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p)
{
    cudaError_t e = cudaErrorInvalidValue;
    // the benchmark shape gets its activations as compile-time constants
    if (c.n_layers == 5 && c.dtype == MLP_F16 && c.hidden_act == MLP_ACT_LEAKY_RELU && c.output_act == MLP_ACT_IDENTITY)
        return launch_narrow_cs<5, MLP_F16, MLP_ACT_LEAKY_RELU, MLP_ACT_IDENTITY, 2, 2, true, 32>(st, ws, p);
#define MLPB200_NARROW32(NL_) \
    if (c.n_layers == NL_) e = c.dtype == MLP_BF16 ? launch_narrow_cs<NL_, MLP_BF16, -1, -1, 2, 2, false, 32>(st, ws, p) \
                                                   : launch_narrow_cs<NL_, MLP_F16, -1, -1, 2, 2, false, 32>(st, ws, p);
    MLPB200_NARROW32(2) MLPB200_NARROW32(3) MLPB200_NARROW32(4) MLPB200_NARROW32(5)
#undef MLPB200_NARROW32
    return e;
}
#endif

#if MLPB200_NARROW_PART == 2
// The two 64-wide benchmark shapes with their activations as compile-time constants.
cudaError_t launch_narrow_named(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p)
{
    if (c.n_layers == 5) return launch_narrow<5, MLP_F16, MLP_ACT_LEAKY_RELU, MLP_ACT_IDENTITY>(st, ws, p);
    // ReLU, four layers, few outputs: two tiles in flight per CTA (two column groups each)
    if (c.dims[4] <= narrow::HMAX / 2 && p.n_tiles > (uint32_t)ws->sm_count)
        return launch_narrow_cs<4, MLP_F16, MLP_ACT_RELU, MLP_ACT_SIGMOID, 2, 2, true>(st, ws, p);
    return launch_narrow<4, MLP_F16, MLP_ACT_RELU, MLP_ACT_SIGMOID>(st, ws, p);
}
#endif

#if MLPB200_NARROW_PART == 3
// Any ReLU network of up to four layers with few outputs: two tiles in flight per CTA.
cudaError_t launch_narrow_relu2(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p)
{
    cudaError_t e = cudaErrorInvalidValue;
#define MLPB200_NARROW2(NL_) \
    if (c.n_layers == NL_) e = c.dtype == MLP_BF16 ? launch_narrow_cs<NL_, MLP_BF16, MLP_ACT_RELU, -1, 2, 2, true>(st, ws, p) \
                                                   : launch_narrow_cs<NL_, MLP_F16, MLP_ACT_RELU, -1, 2, 2, true>(st, ws, p);
    MLPB200_NARROW2(2) MLPB200_NARROW2(3) MLPB200_NARROW2(4)
#undef MLPB200_NARROW2
    return e;
}
#endif

#if MLPB200_NARROW_PART >= 4
// One tile in flight, activations chosen at run time: layer counts 2..5 in either 16-bit format.  Part 4
// builds bf16 with 2 or 3 layers, part 5 bf16 with 4 or 5, parts 6 and 7 the same for fp16.
#define MLPB200_NARROW(NL_, FMT_) if (c.n_layers == NL_ && c.dtype == FMT_) return launch_narrow<NL_, FMT_, -1, -1>(st, ws, p);
#if MLPB200_NARROW_PART == 4
cudaError_t launch_narrow_generic_a(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p)
{
    MLPB200_NARROW(2, MLP_BF16) MLPB200_NARROW(3, MLP_BF16)
    return cudaErrorInvalidValue;
}
#elif MLPB200_NARROW_PART == 5
cudaError_t launch_narrow_generic_b(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p)
{
    MLPB200_NARROW(4, MLP_BF16) MLPB200_NARROW(5, MLP_BF16)
    return cudaErrorInvalidValue;
}
#elif MLPB200_NARROW_PART == 6
cudaError_t launch_narrow_generic_c(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p)
{
    MLPB200_NARROW(2, MLP_F16) MLPB200_NARROW(3, MLP_F16)
    return cudaErrorInvalidValue;
}
#else
cudaError_t launch_narrow_generic_d(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p)
{
    MLPB200_NARROW(4, MLP_F16) MLPB200_NARROW(5, MLP_F16)
    return cudaErrorInvalidValue;
}
#endif
#undef MLPB200_NARROW
#endif

#if MLPB200_NARROW_PART == 0
cudaError_t launch_narrow_generic_a(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p);
cudaError_t launch_narrow_generic_b(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p);
cudaError_t launch_narrow_generic_c(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p);
cudaError_t launch_narrow_generic_d(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const narrow::Params& p);

// Picks the build of the kernel for the shape: padded width, tiles in flight, column split, activations.
// The builds are keyed by the operand format; the kernel itself reads the storage type from its parameters.
static cudaError_t launch_narrow_any(cudaStream_t st, TcWorkspace* ws, const MlpConfig& real, const narrow::Params& p)
{
    MlpConfig c = real;
    if (c.operand_dtype) c.dtype = c.operand_dtype;
    bool fits32 = c.dims[c.n_layers] <= 16;
    for (int l = 0; l <= c.n_layers; ++l) fits32 = fits32 && c.dims[l] <= 32;
    if (fits32) return launch_narrow_fits32(st, ws, c, p);
    if (c.n_layers == 5 && c.dtype == MLP_F16 && c.hidden_act == MLP_ACT_LEAKY_RELU && c.output_act == MLP_ACT_IDENTITY)
        return launch_narrow_named(st, ws, c, p);
    if (c.n_layers == 4 && c.dtype == MLP_F16 && c.hidden_act == MLP_ACT_RELU && c.output_act == MLP_ACT_SIGMOID)
        return launch_narrow_named(st, ws, c, p);
    if (c.hidden_act == MLP_ACT_RELU && c.n_layers >= 2 && c.n_layers <= 4 && c.dims[c.n_layers] <= narrow::HMAX / 2 &&
        p.n_tiles > (uint32_t)ws->sm_count)
        return launch_narrow_relu2(st, ws, c, p);
    if (c.dtype == MLP_BF16) return c.n_layers <= 3 ? launch_narrow_generic_a(st, ws, c, p) : launch_narrow_generic_b(st, ws, c, p);
    return c.n_layers <= 3 ? launch_narrow_generic_c(st, ws, c, p) : launch_narrow_generic_d(st, ws, c, p);
}

cudaError_t launch_forward_narrow(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const MlpForwardParams& a,
                                  int* launches, std::string* err)
{
    if (!tc_train_narrow_supported(c)) { if (err) *err = "shape not built for the narrow tensor-core path"; return cudaErrorInvalidValue; }
    if (a.count == 0) return cudaSuccess;
    narrow::Params p;
    p.cfg = c;
    p.net = (const MlpLayerPointers*)a.networkBuffer;
    p.loss_words = nullptr;
    p.status = ws->status;
    p.inputs = (const void*)a.inputs;
    p.targets = nullptr;
    p.input_grads = nullptr;
    p.outputs = (float*)a.outputs;
    p.count = a.count;
    p.n_tiles = (a.count + narrow::TS - 1) / narrow::TS;
    *launches += 1;
    return launch_narrow_any(st, ws, c, p);
}

cudaError_t launch_learn_gradient_narrow(cudaStream_t st, TcWorkspace* ws, const MlpConfig& c, const MlpLearnGradParamsEx& a,
                                         int* launches, std::string* err, float* input_grads)
{
    if (!tc_train_narrow_supported(c)) { if (err) *err = "shape not built for the narrow tensor-core path"; return cudaErrorInvalidValue; }
    if (a.count == 0) return cudaSuccess;
    narrow::Params p;
    p.cfg = c;
    p.net = (const MlpLayerPointers*)a.networkBuffer;
    p.loss_words = (uint32_t*)a.lossBuffer;
    p.status = ws->status;
    p.inputs = (const void*)a.inputs;
    p.targets = (const void*)a.targets;
    p.input_grads = input_grads;
    p.outputs = nullptr;
    p.count = a.count;
    p.n_tiles = (a.count + narrow::TS - 1) / narrow::TS;
    *launches += 1;
    return launch_narrow_any(st, ws, c, p);
}

#endif  // part 0

}  // namespace mlpb200
