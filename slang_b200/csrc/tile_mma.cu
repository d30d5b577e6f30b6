// Cooperative-matrix multiply-add D = A . B + C as a stand-alone entry point on the tcgen05 tensor cores.
//
// What the reference does: linalg::coopMatMulAdd lowers on CUDA to Slang_CUDA_WMMA::coopMatMulAdd, a 16x16x16
// tile per warp built from two mma.sync.m16n8k16 (prelude/slang-cuda-prelude.h:8145-8642): f16 and bf16 inputs
// with f16/f32 accumulators, s8/u8 with an s32 accumulator (wrapping or .satfinite), e4m3/e5m2 with f32/f16.
//
// Here: one CTA per 128 rows of one problem.  The accumulator lives in tensor memory and is preloaded with C
// (tcgen05.st), so the sum starts from C like the reference's accumulator fragment; A and B go to shared memory
// K-major in 128-byte swizzled panels (zero padded to whole 32-byte K steps and 16 columns), whatever their
// layout in global memory; one thread issues tcgen05.mma of kind f16, i8 or f8f6f4 per 32 bytes of K.
// Every wait is bounded and reports through the device status word.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string>

#include "../../include/slang_b200_tile_mma.h"
#include "abi_internal.h"
#include "tc_host.h"
#include "tc_ptx.cuh"

namespace mlpb200 {
namespace tile {

using namespace ptx;

constexpr uint32_t kStatusTile = 0x4000u;
constexpr int kPanelBytes = 128;   // bytes of K per shared-memory panel row (the swizzle span)

struct Params {
    const uint8_t* a;
    const uint8_t* b;
    const uint8_t* c;
    uint8_t* d;
    int m, n, k;
    int a_col, b_col, cd_col;      // 1: column-major
    long long lda, ldb, ldcd;
    long long stride_a, stride_b, stride_cd;
    int es;                        // bytes per element of A and B
    int acc_half;                  // C and D are half (the sum is fp32)
    int np;                        // N rounded up to a multiple of 16
    uint32_t idesc;
    uint32_t tmem_cols;
    uint32_t* status;
};

// Byte offset of byte kb of row r in a [rows][128-byte] K-major panel with the 128-byte swizzle.
__device__ __forceinline__ uint32_t panel_offset(int r, int kb)
{
    return (uint32_t)r * 128u + (uint32_t)((((kb >> 4) ^ (r & 7)) << 4) | (kb & 15));
}

// KIND: 0 = kind::f16 (f16 / bf16), 1 = kind::i8 (s8 / u8), 2 = kind::f8f6f4 (e4m3 / e5m2)
template <int KIND>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc)
{
    if constexpr (KIND == 0)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc) : "memory");
    else if constexpr (KIND == 1)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc) : "memory");
}

template <int KIND>
__global__ void __launch_bounds__(128, 1) tile_mma_kernel(const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sa = smem;                          // [128 rows][128 bytes]
    uint8_t* sb = smem + 128 * kPanelBytes;      // [np rows][128 bytes]
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_ptr;
    __shared__ uint32_t abort_word;
    volatile uint32_t* abort_flag = &abort_word;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * 128;
    const long long prob = blockIdx.y;
    const uint8_t* A = p.a + prob * p.stride_a * p.es;
    const uint8_t* B = p.b + prob * p.stride_b * p.es;
    const int cd_bytes = p.acc_half ? 2 : 4;
    const uint8_t* C = p.c ? p.c + prob * p.stride_cd * cd_bytes : nullptr;
    uint8_t* D = p.d + prob * p.stride_cd * cd_bytes;

    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_word = 0u;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_ptr, p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_ptr;
    const int r = threadIdx.x;                   // the accumulator row (tensor-memory lane) of this thread
    const int grow = row0 + r;
    const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16);

    // ---- the accumulator starts as C (zero where C is absent or the row / column is padding) ----
    for (int c0 = 0; c0 < p.np; c0 += 16) {
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            v[i] = 0u;
            const int col = c0 + i;
            if (C && grow < p.m && col < p.n) {
                const long long idx = p.cd_col ? (long long)col * p.ldcd + grow : (long long)grow * p.ldcd + col;
                v[i] = p.acc_half ? __float_as_uint(__half2float(((const __half*)C)[idx])) : ((const uint32_t*)C)[idx];
            }
        }
        tmem_st_32x16(t_row + (uint32_t)c0, v);
    }
    tmem_st_wait();

    const int kbytes = p.k * p.es;
    const int n_panels = (kbytes + kPanelBytes - 1) / kPanelBytes;
    bool ok = true;
    for (int pn = 0; pn < n_panels && ok; ++pn) {
        const int kb0 = pn * kPanelBytes;
        const int kb_here = min(kPanelBytes, kbytes - kb0);
        const int kb_pad = (kb_here + 31) & ~31;     // whole K steps of 32 bytes, zero filled
        // ---- A panel: rows of this block, B panel: one row per output column ----
        for (int idx = threadIdx.x; idx < 128 * (kb_pad / p.es); idx += 128) {
            const int rr = idx / (kb_pad / p.es), ke = idx % (kb_pad / p.es);
            const int kk = kb0 / p.es + ke;
            const int gr = row0 + rr;
            uint32_t v = 0;
            if (gr < p.m && kk < p.k) {
                const long long gi = p.a_col ? (long long)kk * p.lda + gr : (long long)gr * p.lda + kk;
                v = p.es == 2 ? ((const uint16_t*)A)[gi] : A[gi];
            }
            if (p.es == 2) *(uint16_t*)(sa + panel_offset(rr, ke * 2)) = (uint16_t)v;
            else sa[panel_offset(rr, ke)] = (uint8_t)v;
        }
        for (int idx = threadIdx.x; idx < p.np * (kb_pad / p.es); idx += 128) {
            const int col = idx / (kb_pad / p.es), ke = idx % (kb_pad / p.es);
            const int kk = kb0 / p.es + ke;
            uint32_t v = 0;
            if (col < p.n && kk < p.k) {
                const long long gi = p.b_col ? (long long)col * p.ldb + kk : (long long)kk * p.ldb + col;
                v = p.es == 2 ? ((const uint16_t*)B)[gi] : B[gi];
            }
            if (p.es == 2) *(uint16_t*)(sb + panel_offset(col, ke * 2)) = (uint16_t)v;
            else sb[panel_offset(col, ke)] = (uint8_t)v;
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        if (threadIdx.x == 0) {
            // K-major, 128-byte swizzle: groups of eight rows 1024 bytes apart; a K step is 32 bytes in the row
            constexpr uint32_t kHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            const uint32_t a_lo = (smem_u32(sa) & 0x3FFFFu) >> 4, b_lo = (smem_u32(sb) & 0x3FFFFu) >> 4;
            for (int ks = 0; ks < kb_pad / 32; ++ks) {
                const uint64_t da = ((uint64_t)kHi << 32) | (a_lo + (uint32_t)(ks * 2) + (1u << 16));
                const uint64_t db = ((uint64_t)kHi << 32) | (b_lo + (uint32_t)(ks * 2) + (1u << 16));
                umma<KIND>(tmem_base, da, db, p.idesc);
            }
            umma_commit(&bar);
        }
        // the products of this panel have read shared memory (and written the accumulator) when the barrier flips
        ok = mbar_wait(&bar, (uint32_t)pn & 1u, abort_flag, p.status, kStatusTile);
        tc_fence_after();
    }

    // ---- D: the accumulator, row by row ----
    if (ok) {
        for (int c0 = 0; c0 < p.np; c0 += 16) {
            uint32_t v[16];
            tmem_ld_32x16(t_row + (uint32_t)c0, v);
            tmem_ld_wait();
            if (grow < p.m) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int col = c0 + i;
                    if (col < p.n) {
                        const long long idx = p.cd_col ? (long long)col * p.ldcd + grow : (long long)grow * p.ldcd + col;
                        if (p.acc_half) ((__half*)D)[idx] = __float2half_rn(__uint_as_float(v[i]));
                        else ((uint32_t*)D)[idx] = v[i];
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, p.tmem_cols);
    }
    (void)lane;
}

}  // namespace tile
}  // namespace mlpb200

using namespace mlpb200;

extern "C" int32_t mlp_tile_mma(MlpDevice* dev, const MlpTileMmaDesc* t, uint64_t a, uint64_t b, uint64_t c, uint64_t d)
{
    if (!dev || !t || !a || !b || !d) { set_last_error("device, descriptor, a, b and d must be given"); return MLP_E_INVALID_ARG; }
    const bool is_int = t->input_type == MLP_TILE_S8 || t->input_type == MLP_TILE_U8;
    const bool is_f8 = t->input_type == MLP_TILE_E4M3 || t->input_type == MLP_TILE_E5M2;
    const bool is_f16 = t->input_type == MLP_TILE_F16 || t->input_type == MLP_TILE_BF16;
    if (!is_int && !is_f8 && !is_f16) { set_last_error("unknown input type"); return MLP_E_INVALID_ARG; }
    // the accumulator types the reference has for each input type
    const bool acc_ok = is_int ? t->acc_type == MLP_TILE_ACC_S32
                               : (t->acc_type == MLP_TILE_ACC_F32 || (t->acc_type == MLP_TILE_ACC_F16 && t->input_type != MLP_TILE_BF16));
    if (!acc_ok) { set_last_error("accumulator type does not go with the input type"); return MLP_E_INVALID_ARG; }
    if (t->saturate && !is_int) { set_last_error("saturation is for integer inputs"); return MLP_E_INVALID_ARG; }
    if (t->m < 1 || t->n < 1 || t->n > 256 || t->k < 1 || t->count < 1 || t->count > 65535) {
        set_last_error("sizes: m >= 1, 1 <= n <= 256, k >= 1, 1 <= count <= 65535");
        return MLP_E_INVALID_ARG;
    }
    for (int lay : {t->a_layout, t->b_layout, t->cd_layout})
        if (lay != MLP_MATRIX_ROW_MAJOR && lay != MLP_MATRIX_COLUMN_MAJOR) { set_last_error("layouts are row- or column-major"); return MLP_E_INVALID_ARG; }
    const auto ld_ok = [](int layout, long long ld, int rows, int cols) { return ld >= (layout == MLP_MATRIX_ROW_MAJOR ? cols : rows); };
    if (!ld_ok(t->a_layout, t->lda, t->m, t->k) || !ld_ok(t->b_layout, t->ldb, t->k, t->n) || !ld_ok(t->cd_layout, t->ldcd, t->m, t->n)) {
        set_last_error("a leading dimension is smaller than the matrix");
        return MLP_E_INVALID_ARG;
    }
    if (t->count > 1 && (t->stride_a < 0 || t->stride_b < 0 || t->stride_cd <= 0)) { set_last_error("batch strides"); return MLP_E_INVALID_ARG; }

    tile::Params p{};
    p.a = (const uint8_t*)a; p.b = (const uint8_t*)b; p.c = (const uint8_t*)c; p.d = (uint8_t*)d;
    p.m = t->m; p.n = t->n; p.k = t->k;
    p.a_col = t->a_layout == MLP_MATRIX_COLUMN_MAJOR; p.b_col = t->b_layout == MLP_MATRIX_COLUMN_MAJOR; p.cd_col = t->cd_layout == MLP_MATRIX_COLUMN_MAJOR;
    p.lda = t->lda; p.ldb = t->ldb; p.ldcd = t->ldcd;
    p.stride_a = t->stride_a; p.stride_b = t->stride_b; p.stride_cd = t->stride_cd;
    p.es = is_f16 ? 2 : 1;
    p.acc_half = t->acc_type == MLP_TILE_ACC_F16;
    p.np = (t->n + 15) & ~15;
    p.tmem_cols = 32; while (p.tmem_cols < (uint32_t)p.np) p.tmem_cols <<= 1;
    p.status = dev->tc->status;
    // instruction descriptor: accumulator format (bits 4-5: 1 = f32, 2 = s32), input formats (bits 7-9 and 10-12),
    // saturation (bit 3), N / 8 (bits 17-22), M / 16 (bits 24-28); both operands K-major
    uint32_t fmt = 0;
    switch (t->input_type) {
    case MLP_TILE_F16: fmt = 0; break;
    case MLP_TILE_BF16: fmt = 1; break;
    case MLP_TILE_U8: fmt = 0; break;
    case MLP_TILE_S8: fmt = 1; break;
    case MLP_TILE_E4M3: fmt = 0; break;
    case MLP_TILE_E5M2: fmt = 1; break;
    }
    p.idesc = ((is_int ? 2u : 1u) << 4) | (fmt << 7) | (fmt << 10) | (((uint32_t)p.np >> 3) << 17) | ((128u >> 4) << 24) |
              ((is_int && t->saturate) ? (1u << 3) : 0u);

    cudaError_t e = cudaSetDevice(dev->ordinal);
    const size_t smem = 1024 + (size_t)(128 + p.np) * tile::kPanelBytes;
    const dim3 grid((unsigned)((t->m + 127) / 128), (unsigned)t->count);
    if (e == cudaSuccess) {
        auto kern = is_f16 ? tile::tile_mma_kernel<0> : is_int ? tile::tile_mma_kernel<1> : tile::tile_mma_kernel<2>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(1024 + (128 + 256) * tile::kPanelBytes));
        if (e == cudaSuccess) {
            kern<<<grid, 128, smem, dev->stream>>>(p);
            e = cudaGetLastError();
        }
    }
    if (e != cudaSuccess) {
        set_last_error((std::string("tile product launch failed: ") + cudaGetErrorString(e)).c_str());
        return MLP_E_CUDA;
    }
    dev->launches += 1;
    return MLP_OK;
}
