/* CPU oracle of the permutohedral-lattice encoder.  TEST INFRASTRUCTURE ONLY: tests and the benchmark's
 * CPU baseline may load this; the product library must not.
 *
 * Restates source/standard-modules/neural/permuto-encoder.slang and hash-function.slang of the reference
 * for one sequential thread: positions in ascending order, levels in ascending order, vertices k = 0..D
 * in ascending order, plain load-add-store accumulation.  The reverse pass is the hand derivative of the
 * forward pass in that same order (the reference obtains it by automatic differentiation, so its order of
 * additions is not defined by its source; its tests accept 0.1 absolute).
 *
 * Pinning: tests/test_permuto.py checks this file against the known answers of the reference's own tests:
 * 22 hash values (tests/neural/hash-function-test.slang:100-121), the level constants
 * (tests/neural/permuto-encoder-precomputed-constants.slang:38-55), 128 forward values, 32 position
 * gradients and 64 table gradients (tests/neural/permuto-reference-data.slang). */
#include <cmath>
#include <cstdint>
#include <cstring>

#include "../include/slang_b200_permuto.h"

namespace {

typedef _Float16 hf;

// ---- PCG32 (hash-function.slang:15-63) ----------------------------------------------------------
struct Pcg32 {
    uint64_t state, inc;
    static constexpr uint64_t kMult = 0x5851f42d4c957f2dULL;
    explicit Pcg32(uint64_t initstate, uint64_t initseq = 1)
    {
        state = 0;
        inc = (initseq << 1) | 1;
        next();
        state += initstate;
        next();
    }
    uint32_t next()
    {
        const uint64_t old = state;
        state = old * kMult + inc;
        const uint32_t xs = uint32_t(((old >> 18) ^ old) >> 27);
        const uint32_t rot = uint32_t(old >> 59);
        return (xs >> rot) | (xs << ((~rot + 1) & 31));
    }
    void advance(uint64_t d)
    {
        uint64_t cur_mult = kMult, cur_plus = inc, acc_mult = 1, acc_plus = 0;
        while (d > 0) {
            if (d & 1) { acc_mult *= cur_mult; acc_plus = acc_plus * cur_mult + cur_plus; }
            cur_plus = (cur_mult + 1) * cur_plus;
            cur_mult *= cur_mult;
            d >>= 1;
        }
        state = acc_mult * state + acc_plus;
    }
};

uint32_t lcg_hash(int dims, const uint32_t* p, const uint32_t* primes)
{
    uint32_t r = 0;
    for (int i = 0; i < dims; ++i) r ^= p[i] * primes[i];
    return r;
}

uint32_t base_convert_hash(int dims, const uint32_t* p)
{
    uint32_t k = 0;
    for (int d = 0; d < dims; ++d) { k += p[d]; k *= 2531011u; }
    return k;
}

uint32_t rng_hash(int dims, const uint32_t* p, uint32_t seed = 1337)
{
    const int bits = 64 / dims;
    uint64_t step = 0;
    for (int i = 0; i < dims; ++i) step ^= uint64_t(p[i]) << (i * bits);
    Pcg32 rng(seed);
    rng.advance(step);
    return rng.next();
}

// ---- one level of one position -------------------------------------------------------------------
struct Simplex {
    float elevated[MLP_PERMUTO_MAX_DIMS + 1];
    int rem0[MLP_PERMUTO_MAX_DIMS + 1];
    int rank[MLP_PERMUTO_MAX_DIMS + 1];
    float bary[MLP_PERMUTO_MAX_DIMS + 2];
};

void locate(int D, const float* pos, const MlpPermutoLevelInfo& li, Simplex& s)
{
    // elevate (permuto-encoder.slang:70-86)
    float sum = 0.0f;
    for (int dim = D - 1; dim >= 0; --dim) {
        const float cf = (pos[dim] + li.shifts_per_dim[dim]) * li.scales_per_dim[dim];
        s.elevated[dim + 1] = sum - float(dim + 1) * cf;
        sum += cf;
    }
    s.elevated[0] = sum;
    // closest remainder-0 point and ranks (permuto-encoder.slang:93-155)
    const float inv = 1.0f / float(D + 1);
    int isum = 0;
    for (int dim = 0; dim <= D; ++dim) {
        const float v = s.elevated[dim] * inv;
        const float up = std::ceil(v) * float(D + 1), down = std::floor(v) * float(D + 1);
        s.rem0[dim] = (up - s.elevated[dim] < s.elevated[dim] - down) ? int(up) : int(down);
        isum += s.rem0[dim];
        s.rank[dim] = 0;
    }
    isum /= (D + 1);
    for (int dim = 0; dim < D; ++dim) {
        const float di = s.elevated[dim] - float(s.rem0[dim]);
        for (int other = dim + 1; other <= D; ++other) {
            if (di < s.elevated[other] - float(s.rem0[other])) s.rank[dim]++;
            else s.rank[other]++;
        }
    }
    for (int dim = 0; dim <= D; ++dim) {
        s.rank[dim] += isum;
        if (s.rank[dim] < 0) { s.rank[dim] += D + 1; s.rem0[dim] += D + 1; }
        else if (s.rank[dim] > D) { s.rank[dim] -= D + 1; s.rem0[dim] -= D + 1; }
    }
    // barycentric coordinates (permuto-encoder.slang:164-184)
    for (int i = 0; i < D + 2; ++i) s.bary[i] = 0.0f;
    for (int dim = 0; dim <= D; ++dim) {
        const float delta = (s.elevated[dim] - float(s.rem0[dim])) * inv;
        s.bary[D - s.rank[dim]] += delta;
        s.bary[D + 1 - s.rank[dim]] -= delta;
    }
    s.bary[0] += 1.0f + s.bary[D + 1];
}

uint32_t vertex_index(int D, const Simplex& s, int k, const MlpPermutoLevelInfo& li, int F)
{
    uint32_t key[MLP_PERMUTO_MAX_DIMS];
    for (int dim = 0; dim < D; ++dim) {
        key[dim] = uint32_t(s.rem0[dim] + k);
        if (s.rank[dim] > D - k) key[dim] -= uint32_t(D + 1);
    }
    return li.table_offset * uint32_t(F) + (base_convert_hash(D, key) % li.table_size) * uint32_t(F);
}

template <typename T>
void encode_all(const MlpPermutoConfig& c, const float* positions, const T* table, T* out, uint32_t count)
{
    const int D = c.dims, F = c.features_per_entry, L = c.n_levels;
    for (uint32_t n = 0; n < count; ++n) {
        T* row = out + size_t(n) * L * F;
        for (int l = 0; l < L; ++l) {
            const MlpPermutoLevelInfo& li = c.levels[l];
            T* o = row + li.level_index * F;
            for (int f = 0; f < F; ++f) o[f] = T(0);
            if (float(li.level_index) >= c.max_level + 1e-3f) continue;
            Simplex s;
            locate(D, positions + size_t(n) * D, li, s);
            for (int k = 0; k <= D; ++k) {
                const uint32_t idx = vertex_index(D, s, k, li, F);
                const T w = T(s.bary[k]);
                for (int f = 0; f < F; ++f) o[f] = T(o[f] + T(w * table[idx + f]));
            }
        }
    }
}

template <typename T>
void backward_all(const MlpPermutoConfig& c, const float* positions, const T* table, const T* d_out, T* d_table,
                  float* d_positions, uint32_t count)
{
    const int D = c.dims, F = c.features_per_entry, L = c.n_levels;
    for (uint32_t n = 0; n < count; ++n) {
        float dpos[MLP_PERMUTO_MAX_DIMS] = {0, 0, 0, 0};
        for (int l = 0; l < L; ++l) {
            const MlpPermutoLevelInfo& li = c.levels[l];
            if (float(li.level_index) >= c.max_level + 1e-3f) continue;
            const T* dy = d_out + size_t(n) * L * F + li.level_index * F;
            Simplex s;
            locate(D, positions + size_t(n) * D, li, s);
            float dbary[MLP_PERMUTO_MAX_DIMS + 2];
            for (int k = 0; k <= D; ++k) {
                const uint32_t idx = vertex_index(D, s, k, li, F);
                const T w = T(s.bary[k]);
                float dw = 0.0f;
                for (int f = 0; f < F; ++f) {
                    d_table[idx + f] = T(d_table[idx + f] + T(w * dy[f]));
                    dw += float(T(table[idx + f] * dy[f]));
                }
                dbary[k] = dw;
            }
            // barycentric[0] += 1 + barycentric[D + 1]
            dbary[D + 1] = dbary[0];
            const float inv = 1.0f / float(D + 1);
            float de[MLP_PERMUTO_MAX_DIMS + 1];
            for (int dim = 0; dim <= D; ++dim)
                de[dim] = (dbary[D - s.rank[dim]] - dbary[D + 1 - s.rank[dim]]) * inv;
            // elevated[0] = sum of all cf; elevated[dim + 1] = (sum of cf of higher dims) - (dim + 1) cf
            float run = de[0];
            for (int dim = 0; dim < D; ++dim) {
                const float dcf = run - float(dim + 1) * de[dim + 1];
                dpos[dim] += dcf * li.scales_per_dim[dim];
                run += de[dim + 1];
            }
        }
        if (d_positions)
            for (int dim = 0; dim < D; ++dim) d_positions[size_t(n) * D + dim] = dpos[dim];
    }
}

}  // namespace

extern "C" {

uint32_t permuto_oracle_grid_hash(int32_t type, int32_t dims, const uint32_t* p)
{
    static const uint32_t prime[7] = {1958374283u, 2654435761u, 805459861u, 3674653429u, 2097192037u, 1434869437u, 2165219737u};
    static const uint32_t coherent[7] = {1u, 2654435761u, 805459861u, 3674653429u, 2097192037u, 1434869437u, 2165219737u};
    static const uint32_t reversed[7] = {2165219737u, 1434869437u, 2097192037u, 3674653429u, 805459861u, 2654435761u, 1958374283u};
    switch (type) {
    case 0: return lcg_hash(dims, p, prime);
    case 1: return lcg_hash(dims, p, coherent);
    case 2: return lcg_hash(dims, p, reversed);
    case 3: return rng_hash(dims, p);
    case 4: return base_convert_hash(dims, p);
    default: return 0;
    }
}

int permuto_oracle_prepare(int32_t dims, int32_t features, int32_t log2_size, int32_t n_levels, float base_scale,
                           float log2_per_level_scale, float max_level_ratio, uint32_t seed, int32_t dtype,
                           MlpPermutoConfig* out)
{
    if (dims < 1 || dims > MLP_PERMUTO_MAX_DIMS || n_levels < 1 || n_levels > MLP_PERMUTO_MAX_LEVELS) return -1;
    std::memset(out, 0, sizeof *out);
    out->dims = dims; out->features_per_entry = features; out->log2_hashmap_size = log2_size; out->n_levels = n_levels;
    out->dtype = dtype;
    out->max_level = max_level_ratio * float(n_levels);
    const uint32_t size = 1u << log2_size;
    for (int l = 0; l < n_levels; ++l) {
        MlpPermutoLevelInfo& li = out->levels[l];
        li.level_index = uint32_t(l);
        li.table_size = size;
        li.table_offset = uint32_t(l) * size;
        li.scale = base_scale * std::exp2(float(l) * log2_per_level_scale);
        Pcg32 rng(seed);
        rng.advance(uint64_t(l) * uint64_t(dims));
        for (int d = 0; d < dims; ++d) {
            li.scales_per_dim[d] = li.scale * (1.0f / std::sqrt(float((d + 1) * (d + 2))));
            const float r = float(rng.next()) * (1.0f / 4294967296.0f);
            li.shifts_per_dim[d] = r * 10.0f - 5.0f;
        }
    }
    return 0;
}

int permuto_oracle_encode(const MlpPermutoConfig* c, const float* positions, const void* table, void* out, uint32_t count)
{
    if (c->dtype == MLP_F32) encode_all<float>(*c, positions, (const float*)table, (float*)out, count);
    else if (c->dtype == MLP_F16) encode_all<hf>(*c, positions, (const hf*)table, (hf*)out, count);
    else return -1;
    return 0;
}

int permuto_oracle_backward(const MlpPermutoConfig* c, const float* positions, const void* table, const void* d_out,
                            void* d_table, float* d_positions, uint32_t count)
{
    if (c->dtype == MLP_F32) backward_all<float>(*c, positions, (const float*)table, (const float*)d_out, (float*)d_table, d_positions, count);
    else if (c->dtype == MLP_F16) backward_all<hf>(*c, positions, (const hf*)table, (const hf*)d_out, (hf*)d_table, d_positions, count);
    else return -1;
    return 0;
}

}  // extern "C"
