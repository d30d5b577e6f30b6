// Permutohedral-lattice hash encoder (include/slang_b200_permuto.h): host-side preparation of the level
// constants, the grid hashes, and the encode / reverse kernels.
//
// Follows PermutoEncoder of the reference's neural module (source/standard-modules/neural/
// permuto-encoder.slang:55-330) and its hashes (hash-function.slang:15-145).  One thread handles one
// (position, level) pair, levels fastest, so that the threads of a warp write one contiguous piece of an
// output row and read their vertices' features with one vector load each.  The reverse pass adds
// weight * upstream gradient into the gradient table with vector reductions (one red per vertex for up to
// four fp32 / eight fp16 features) and sums the levels' position gradients in ascending level order inside
// the block.  Compiled with -fmad=false: every multiply and add rounds on its own, which makes the forward
// pass bit-identical to a sequential CPU evaluation of the same expressions.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <string>

#include "../../include/slang_b200_permuto.h"
#include "abi_internal.h"

using namespace mlpb200;

namespace {

// ---- PCG32 and the hashes (host and device) -------------------------------------------------------
struct Pcg32 {
    uint64_t state, inc;
    __host__ __device__ explicit Pcg32(uint64_t initstate, uint64_t initseq = 1)
    {
        state = 0;
        inc = (initseq << 1) | 1;
        next();
        state += initstate;
        next();
    }
    __host__ __device__ uint32_t next()
    {
        const uint64_t old = state;
        state = old * 0x5851f42d4c957f2dULL + inc;
        const uint32_t xs = uint32_t(((old >> 18) ^ old) >> 27), rot = uint32_t(old >> 59);
        return (xs >> rot) | (xs << ((~rot + 1) & 31));
    }
    // Jumps the generator ahead by delta draws in O(log delta).
    __host__ __device__ void advance(uint64_t delta)
    {
        uint64_t m = 0x5851f42d4c957f2dULL, p = inc, am = 1, ap = 0;
        for (; delta; delta >>= 1) {
            if (delta & 1) { am *= m; ap = ap * m + p; }
            p = (m + 1) * p;
            m *= m;
        }
        state = am * state + ap;
    }
};

template <int D>
__host__ __device__ inline uint32_t base_convert_hash(const uint32_t* key)
{
    uint32_t k = 0;
#pragma unroll
    for (int d = 0; d < D; ++d) { k += key[d]; k *= 2531011u; }
    return k;
}

uint32_t host_grid_hash(int type, int dims, const uint32_t* p)
{
    static const uint32_t primes[3][7] = {
        {1958374283u, 2654435761u, 805459861u, 3674653429u, 2097192037u, 1434869437u, 2165219737u},
        {1u, 2654435761u, 805459861u, 3674653429u, 2097192037u, 1434869437u, 2165219737u},
        {2165219737u, 1434869437u, 2097192037u, 3674653429u, 805459861u, 2654435761u, 1958374283u}};
    if (dims < 1 || dims > 7) return 0;
    if (type >= 0 && type <= 2) {
        uint32_t r = 0;
        for (int i = 0; i < dims; ++i) r ^= p[i] * primes[type][i];
        return r;
    }
    if (type == 3) {
        const int bits = 64 / dims;
        uint64_t step = 0;
        for (int i = 0; i < dims; ++i) step ^= uint64_t(p[i]) << (i * bits);
        Pcg32 rng(1337);
        rng.advance(step);
        return rng.next();
    }
    if (type == 4) {
        uint32_t k = 0;
        for (int d = 0; d < dims; ++d) { k += p[d]; k *= 2531011u; }
        return k;
    }
    return 0;
}

// ---- element types --------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    __device__ static float from(float v) { return v; }
    __device__ static float to_float(float v) { return v; }
    __device__ static float mul(float a, float b) { return a * b; }
    __device__ static float add(float a, float b) { return a + b; }
};
template <> struct Elem<__half> {
    __device__ static __half from(float v) { return __float2half_rn(v); }
    __device__ static float to_float(__half v) { return __half2float(v); }
    // one rounding per operation, as half arithmetic does
    __device__ static __half mul(__half a, __half b) { return __float2half_rn(__half2float(a) * __half2float(b)); }
    __device__ static __half add(__half a, __half b) { return __float2half_rn(__half2float(a) + __half2float(b)); }
};

template <int F, typename T> struct alignas(sizeof(T) * F) Vec { T v[F]; };

template <int F, typename T>
__device__ inline Vec<F, T> load_vec(const T* p)
{
    return *reinterpret_cast<const Vec<F, T>*>(p);   // F * sizeof(T) is 2..32 bytes and p is aligned to it
}

// Adds F values to F consecutive table slots with as few reductions as the types allow.
template <int F>
__device__ inline void red_add(float* p, const float* v)
{
    if constexpr (F % 4 == 0) {
#pragma unroll
        for (int i = 0; i < F; i += 4) atomicAdd(reinterpret_cast<float4*>(p + i), make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]));
    } else if constexpr (F == 2) {
        atomicAdd(reinterpret_cast<float2*>(p), make_float2(v[0], v[1]));
    } else {
        atomicAdd(p, v[0]);
    }
}
template <int F>
__device__ inline void red_add(__half* p, const __half* v)
{
    if constexpr (F % 2 == 0) {
#pragma unroll
        for (int i = 0; i < F; i += 2) atomicAdd(reinterpret_cast<__half2*>(p + i), __halves2half2(v[i], v[i + 1]));
    } else {
        atomicAdd(p, v[0]);
    }
}

// ---- geometry of one (position, level) ----------------------------------------------------------------
template <int D>
struct Simplex {
    float elevated[D + 1];
    int rem0[D + 1];
    int rank[D + 1];
    float bary[D + 2];
};

template <int D>
__device__ inline void locate(const float* pos, const MlpPermutoLevelInfo& li, Simplex<D>& s)
{
    float sum = 0.0f;
#pragma unroll
    for (int dim = D - 1; dim >= 0; --dim) {
        const float cf = (pos[dim] + li.shifts_per_dim[dim]) * li.scales_per_dim[dim];
        s.elevated[dim + 1] = sum - float(dim + 1) * cf;
        sum += cf;
    }
    s.elevated[0] = sum;
    constexpr float inv = 1.0f / float(D + 1);
    int isum = 0;
#pragma unroll
    for (int dim = 0; dim <= D; ++dim) {
        const float v = s.elevated[dim] * inv;
        const float up = ceilf(v) * float(D + 1), down = floorf(v) * float(D + 1);
        s.rem0[dim] = (up - s.elevated[dim] < s.elevated[dim] - down) ? int(up) : int(down);
        isum += s.rem0[dim];
        s.rank[dim] = 0;
    }
    isum /= (D + 1);
#pragma unroll
    for (int dim = 0; dim < D; ++dim) {
        const float di = s.elevated[dim] - float(s.rem0[dim]);
#pragma unroll
        for (int other = dim + 1; other <= D; ++other) {
            const bool lower = di < s.elevated[other] - float(s.rem0[other]);
            s.rank[dim] += lower ? 1 : 0;
            s.rank[other] += lower ? 0 : 1;
        }
    }
#pragma unroll
    for (int dim = 0; dim <= D; ++dim) {
        s.rank[dim] += isum;
        if (s.rank[dim] < 0) { s.rank[dim] += D + 1; s.rem0[dim] += D + 1; }
        else if (s.rank[dim] > D) { s.rank[dim] -= D + 1; s.rem0[dim] -= D + 1; }
    }
#pragma unroll
    for (int i = 0; i < D + 2; ++i) s.bary[i] = 0.0f;
#pragma unroll
    for (int dim = 0; dim <= D; ++dim) {
        const float delta = (s.elevated[dim] - float(s.rem0[dim])) * inv;
        // rank is 0..D: add to slot D - rank, subtract from slot D + 1 - rank (compile-time slots keep
        // the array in registers)
#pragma unroll
        for (int r = 0; r <= D; ++r)
            if (s.rank[dim] == r) { s.bary[D - r] += delta; s.bary[D + 1 - r] -= delta; }
    }
    s.bary[0] += 1.0f + s.bary[D + 1];
}

template <int D, int F>
__device__ inline uint32_t vertex_index(const Simplex<D>& s, int k, const MlpPermutoLevelInfo& li)
{
    uint32_t key[D];
#pragma unroll
    for (int dim = 0; dim < D; ++dim) {
        key[dim] = uint32_t(s.rem0[dim] + k);
        if (s.rank[dim] > D - k) key[dim] -= uint32_t(D + 1);
    }
    const uint32_t h = base_convert_hash<D>(key);
    // x % 2^k == x & (2^k - 1); the general remainder only for tables that are not a power of two
    const uint32_t slot = (li.table_size & (li.table_size - 1)) == 0 ? (h & (li.table_size - 1)) : (h % li.table_size);
    return (li.table_offset + slot) * uint32_t(F);
}

__device__ inline bool level_live(const MlpPermutoConfig& c, const MlpPermutoLevelInfo& li)
{
    return !(float(li.level_index) >= c.max_level + 1e-3f);
}

// Thread mapping of both kernels: a block of 256 threads is floor(256 / L) positions x L levels, levels
// fastest, so the level threads of a position write one contiguous output row.  The grid is sized to the
// machine and every block walks over position groups with a grid stride; a thread keeps its level for its
// whole life, so it reads its level's constants from the kernel parameters once.
template <int D, int F, typename T>
__global__ void __launch_bounds__(256)
permuto_encode_kernel(const __grid_constant__ MlpPermutoConfig c, const float* __restrict__ positions,
                      const T* __restrict__ table, T* __restrict__ out, uint32_t count)
{
    const uint32_t L = uint32_t(c.n_levels);
    const uint32_t per_block = 256u / L;
    const uint32_t local = threadIdx.x / L, l = threadIdx.x - local * L;
    if (local >= per_block) return;
    const MlpPermutoLevelInfo li = c.levels[l];
    const bool live = level_live(c, li);
    const uint64_t row = uint64_t(L) * F;
    for (uint64_t n = uint64_t(blockIdx.x) * per_block + local; n < count; n += uint64_t(gridDim.x) * per_block) {
        T acc[F];
#pragma unroll
        for (int f = 0; f < F; ++f) acc[f] = Elem<T>::from(0.0f);
        if (live) {
            float pos[D];
#pragma unroll
            for (int d = 0; d < D; ++d) pos[d] = positions[n * D + d];
            Simplex<D> s;
            locate<D>(pos, li, s);
            Vec<F, T> feat[D + 1];
#pragma unroll
            for (int k = 0; k <= D; ++k) feat[k] = load_vec<F, T>(table + vertex_index<D, F>(s, k, li));
#pragma unroll
            for (int k = 0; k <= D; ++k) {
                const T w = Elem<T>::from(s.bary[k]);
#pragma unroll
                for (int f = 0; f < F; ++f) acc[f] = Elem<T>::add(acc[f], Elem<T>::mul(w, feat[k].v[f]));
            }
        }
        Vec<F, T> o;
#pragma unroll
        for (int f = 0; f < F; ++f) o.v[f] = acc[f];
        *reinterpret_cast<Vec<F, T>*>(out + n * row + uint64_t(li.level_index) * F) = o;
    }
}

// The level-0 thread of a position adds the level threads' position-gradient terms in ascending level
// order: by warp shuffles when a warp holds whole positions (L divides 32), through shared memory otherwise.
template <int D, int F, typename T>
__global__ void __launch_bounds__(256)
permuto_backward_kernel(const __grid_constant__ MlpPermutoConfig c, const float* __restrict__ positions,
                        const T* __restrict__ table, const T* __restrict__ d_out, T* __restrict__ d_table,
                        float* __restrict__ d_positions, uint32_t count)
{
    __shared__ float s_dpos[256 * D];
    __shared__ MlpPermutoLevelInfo s_levels[MLP_PERMUTO_MAX_LEVELS];
    const uint32_t L = uint32_t(c.n_levels);
    const uint32_t per_block = 256u / L;
    const uint32_t local = threadIdx.x / L, l = threadIdx.x - local * L;
    // This kernel runs as many short-lived blocks (the reductions retire faster that way), so the level
    // constants go through shared memory: a kernel parameter indexed per lane is fetched once per
    // distinct level of the warp.
    {
        constexpr int kWords = sizeof(MlpPermutoLevelInfo) / 4;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(c.levels);
        uint32_t* dst = reinterpret_cast<uint32_t*>(s_levels);
        for (uint32_t i = threadIdx.x; i < L * kWords; i += blockDim.x) dst[i] = src[i];
        __syncthreads();
    }
    const MlpPermutoLevelInfo li = s_levels[l];
    const bool live = level_live(c, li);
    const uint64_t row = uint64_t(L) * F;
    for (uint64_t base = uint64_t(blockIdx.x) * per_block; base < count; base += uint64_t(gridDim.x) * per_block) {
        const uint64_t n = base + local;
        const bool active = local < per_block && n < count;
        float dpos[D];
#pragma unroll
        for (int d = 0; d < D; ++d) dpos[d] = 0.0f;
        if (active && live) {
            float pos[D];
#pragma unroll
            for (int d = 0; d < D; ++d) pos[d] = positions[n * D + d];
            Simplex<D> s;
            locate<D>(pos, li, s);
            const Vec<F, T> dy = load_vec<F, T>(d_out + n * row + uint64_t(li.level_index) * F);
            float dbary[D + 2];
#pragma unroll
            for (int k = 0; k <= D; ++k) {
                const uint32_t idx = vertex_index<D, F>(s, k, li);
                const Vec<F, T> feat = load_vec<F, T>(table + idx);
                const T w = Elem<T>::from(s.bary[k]);
                T term[F];
                float dw = 0.0f;
#pragma unroll
                for (int f = 0; f < F; ++f) {
                    term[f] = Elem<T>::mul(w, dy.v[f]);
                    dw += Elem<T>::to_float(Elem<T>::mul(feat.v[f], dy.v[f]));
                }
                red_add<F>(d_table + idx, term);
                dbary[k] = dw;
            }
            if (d_positions) {
                dbary[D + 1] = dbary[0];
                constexpr float inv = 1.0f / float(D + 1);
                float de[D + 1];
#pragma unroll
                for (int dim = 0; dim <= D; ++dim) {
                    float plus = 0.0f, minus = 0.0f;
#pragma unroll
                    for (int r = 0; r <= D; ++r)
                        if (s.rank[dim] == r) { plus = dbary[D - r]; minus = dbary[D + 1 - r]; }
                    de[dim] = (plus - minus) * inv;
                }
                float run = de[0];
#pragma unroll
                for (int dim = 0; dim < D; ++dim) {
                    const float dcf = run - float(dim + 1) * de[dim + 1];
                    dpos[dim] = dcf * li.scales_per_dim[dim];
                    run += de[dim + 1];
                }
            }
        }
        if (d_positions) {   // uniform over the block
            if ((32u % L) == 0) {
                // the level threads of a position sit in one warp: the level-0 lane pulls the others' terms
                // in ascending level order (every lane runs the shuffles; lanes past the batch carry zeros)
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    float acc = 0.0f + dpos[d];
                    for (uint32_t j = 1; j < L; ++j) acc += __shfl_down_sync(0xffffffffu, dpos[d], j);
                    if (active && l == 0) d_positions[n * D + d] = acc;
                }
            } else {
#pragma unroll
                for (int d = 0; d < D; ++d) s_dpos[threadIdx.x * D + d] = dpos[d];
                __syncthreads();
                if (active && l == 0) {
#pragma unroll
                    for (int d = 0; d < D; ++d) {
                        float acc = 0.0f;
                        for (uint32_t j = 0; j < L; ++j) acc += s_dpos[(threadIdx.x + j) * D + d];
                        d_positions[n * D + d] = acc;
                    }
                }
                __syncthreads();
            }
        }
    }
}

bool config_ok(const MlpPermutoConfig* c, std::string* why)
{
    if (!c) { *why = "null config"; return false; }
    if (c->dims < 1 || c->dims > MLP_PERMUTO_MAX_DIMS) { *why = "dims out of range (1..4)"; return false; }
    if (c->features_per_entry != 1 && c->features_per_entry != 2 && c->features_per_entry != 4 && c->features_per_entry != 8) {
        *why = "features_per_entry must be 1, 2, 4 or 8"; return false;
    }
    if (c->n_levels < 1 || c->n_levels > MLP_PERMUTO_MAX_LEVELS) { *why = "n_levels out of range (1..32)"; return false; }
    if (c->log2_hashmap_size < 0 || c->log2_hashmap_size > 26) { *why = "log2_hashmap_size out of range (0..26)"; return false; }
    if (c->dtype != MLP_F32 && c->dtype != MLP_F16) { *why = "dtype must be MLP_F32 or MLP_F16"; return false; }
    uint64_t values = 0;
    for (int l = 0; l < c->n_levels; ++l) {
        const MlpPermutoLevelInfo& li = c->levels[l];
        if (li.table_size == 0) { *why = "a level has an empty table"; return false; }
        if (li.level_index >= uint32_t(c->n_levels)) { *why = "level_index out of range"; return false; }
        values = (uint64_t(li.table_offset) + li.table_size) * uint64_t(c->features_per_entry);
        if (values > (uint64_t(1) << 32)) { *why = "table larger than 2^32 values"; return false; }
    }
    return true;
}

template <int D, int F, typename T>
cudaError_t run(bool backward, cudaStream_t st, const MlpPermutoConfig& c, uint64_t positions, uint64_t table, uint64_t out,
                uint64_t d_table, uint64_t d_positions, uint32_t count)
{
    const uint32_t L = uint32_t(c.n_levels);
    const uint32_t per_block = 256u / L;
    const uint64_t groups = (uint64_t(count) + per_block - 1) / per_block;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int resident = 0;   // blocks of this kernel that fit an SM at once
    if (!backward) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, permuto_encode_kernel<D, F, T>, 256, 0);
    else cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, permuto_backward_kernel<D, F, T>, 256, 0);
    if (resident < 1) resident = 1;
    // encode: one wave of blocks that walk the positions; reverse: up to 64 waves of short blocks
    const unsigned grid = (unsigned)std::min<uint64_t>(groups, uint64_t(sms) * resident * (backward ? 64 : 1));
    if (!backward) {
        permuto_encode_kernel<D, F, T><<<grid, 256, 0, st>>>(
            c, (const float*)positions, (const T*)table, (T*)out, count);
    } else {
        permuto_backward_kernel<D, F, T><<<grid, 256, 0, st>>>(
            c, (const float*)positions, (const T*)table, (const T*)out, (T*)d_table, (float*)d_positions, count);
    }
    return cudaGetLastError();
}

template <int D, typename T>
cudaError_t run_f(bool backward, cudaStream_t st, const MlpPermutoConfig& c, uint64_t a, uint64_t b, uint64_t o, uint64_t dt,
                  uint64_t dp, uint32_t n)
{
    switch (c.features_per_entry) {
    case 1: return run<D, 1, T>(backward, st, c, a, b, o, dt, dp, n);
    case 2: return run<D, 2, T>(backward, st, c, a, b, o, dt, dp, n);
    case 4: return run<D, 4, T>(backward, st, c, a, b, o, dt, dp, n);
    default: return run<D, 8, T>(backward, st, c, a, b, o, dt, dp, n);
    }
}

template <typename T>
cudaError_t run_d(bool backward, cudaStream_t st, const MlpPermutoConfig& c, uint64_t a, uint64_t b, uint64_t o, uint64_t dt,
                  uint64_t dp, uint32_t n)
{
    switch (c.dims) {
    case 1: return run_f<1, T>(backward, st, c, a, b, o, dt, dp, n);
    case 2: return run_f<2, T>(backward, st, c, a, b, o, dt, dp, n);
    case 3: return run_f<3, T>(backward, st, c, a, b, o, dt, dp, n);
    default: return run_f<4, T>(backward, st, c, a, b, o, dt, dp, n);
    }
}

int32_t launch(bool backward, MlpDevice* d, const MlpPermutoConfig* c, uint64_t positions, uint64_t table, uint64_t out,
               uint64_t d_table, uint64_t d_positions, uint32_t count)
{
    std::string why;
    if (!d) { set_last_error("null device"); return MLP_E_INVALID_ARG; }
    if (!config_ok(c, &why)) { set_last_error(("bad encoder config: " + why).c_str()); return MLP_E_INVALID_ARG; }
    if (count == 0) return MLP_OK;
    if (!positions || !table || !out || (backward && !d_table)) { set_last_error("null device address"); return MLP_E_INVALID_ARG; }
    const uint64_t vec = uint64_t(c->features_per_entry) * (c->dtype == MLP_F32 ? 4 : 2);
    if ((table % vec) || (out % vec) || (backward && (d_table % vec)) || (positions % 4) || (d_positions % 4)) {
        set_last_error("tables and feature rows must be aligned to features_per_entry elements");
        return MLP_E_INVALID_ARG;
    }
    cudaError_t e = cudaSetDevice(d->ordinal);
    if (e == cudaSuccess)
        e = c->dtype == MLP_F32 ? run_d<float>(backward, d->stream, *c, positions, table, out, d_table, d_positions, count)
                                : run_d<__half>(backward, d->stream, *c, positions, table, out, d_table, d_positions, count);
    if (e != cudaSuccess) { set_last_error((std::string("kernel launch failed: ") + cudaGetErrorString(e)).c_str()); return MLP_E_CUDA; }
    d->launches += 1;
    return MLP_OK;
}

}  // namespace

extern "C" {

uint32_t mlp_grid_hash(int32_t type, int32_t dims, const uint32_t* position_grid)
{
    if (!position_grid) return 0;
    return host_grid_hash(type, dims, position_grid);
}

int32_t mlp_permuto_prepare(int32_t dims, int32_t features_per_entry, int32_t log2_hashmap_size, int32_t n_levels,
                            float base_scale, float log2_per_level_scale, float max_level_ratio, uint32_t seed,
                            int32_t dtype, MlpPermutoConfig* out)
{
    if (!out) { set_last_error("null argument"); return MLP_E_INVALID_ARG; }
    std::memset(out, 0, sizeof *out);
    out->dims = dims;
    out->features_per_entry = features_per_entry;
    out->log2_hashmap_size = log2_hashmap_size;
    out->n_levels = n_levels;
    out->dtype = dtype;
    if (dims < 1 || dims > MLP_PERMUTO_MAX_DIMS || n_levels < 1 || n_levels > MLP_PERMUTO_MAX_LEVELS ||
        log2_hashmap_size < 0 || log2_hashmap_size > 26) {
        set_last_error("bad encoder config: dims, n_levels or log2_hashmap_size out of range");
        return MLP_E_INVALID_ARG;
    }
    out->max_level = max_level_ratio * float(n_levels);
    const uint32_t size = 1u << log2_hashmap_size;
    for (int l = 0; l < n_levels; ++l) {
        MlpPermutoLevelInfo& li = out->levels[l];
        li.level_index = uint32_t(l);
        li.table_size = size;
        li.table_offset = uint32_t(l) * size;
        li.scale = base_scale * exp2f(float(l) * log2_per_level_scale);
        Pcg32 rng(seed);
        rng.advance(uint64_t(l) * uint64_t(dims));   // every level draws its own shifts
        for (int d = 0; d < dims; ++d) {
            li.scales_per_dim[d] = li.scale * (1.0f / sqrtf(float((d + 1) * (d + 2))));
            li.shifts_per_dim[d] = float(rng.next()) * (1.0f / 4294967296.0f) * 10.0f - 5.0f;
        }
    }
    std::string why;
    if (!config_ok(out, &why)) { set_last_error(("bad encoder config: " + why).c_str()); return MLP_E_INVALID_ARG; }
    return MLP_OK;
}

int32_t mlp_permuto_encode(MlpDevice* device, const MlpPermutoConfig* config, uint64_t positions, uint64_t table,
                           uint64_t out, uint32_t count)
{
    return launch(false, device, config, positions, table, out, 0, 0, count);
}

int32_t mlp_permuto_backward(MlpDevice* device, const MlpPermutoConfig* config, uint64_t positions, uint64_t table,
                             uint64_t d_out, uint64_t d_table, uint64_t d_positions, uint32_t count)
{
    return launch(true, device, config, positions, table, d_out, d_table, d_positions, count);
}

}  // extern "C"
