/*
 * CPU oracle for the batched small-MLP training step.  TEST INFRASTRUCTURE ONLY: nothing in the
 * product path may call, link or import this file; tests, the smoke check and the benchmark's CPU
 * baseline use it as the checker.
 *
 * It restates, in plain C++, what the reference's Slang kernels compute when they run on the
 * reference's CPU target:
 *   - execution order: groups, then threads, strictly sequential, so every accumulation into a
 *     gradient buffer happens in ascending sample order, one add at a time
 *     (source/slang/slang-emit-cpp.cpp:2210-2284);
 *   - accumulation: plain load-add-store, as in the software fallbacks of
 *     coopVecOuterProductAccumulate / coopVecReduceSumAccumulate
 *     (source/slang/hlsl.meta.slang:33261-33315, 33344-33351);
 *   - layer math: y = W x + b with W row-major [out][in], the terms added in ascending input order.
 *     MlpConfig.sum_order picks between the two orders the reference itself uses:
 *       MLP_SUM_NEURAL (default): the sum starts at zero, each product is rounded before it is added
 *       and the bias is added after the last term, as InlineVector.linearTransform and the
 *       cooperative-vector software fallback do (source/standard-modules/neural/inline-vector.slang:101-110,
 *       131-132; source/slang/hlsl.meta.slang:32866 and the bias loop after it); dx sums rounded
 *       products from zero (inline-vector.slang:149-159) and dW adds a rounded product
 *       (inline-vector.slang:163-175, hlsl.meta.slang:33266-33274);
 *       MLP_SUM_BIAS_FIRST_FUSED: the example's order, the sum starting from the bias
 *       (examples/mlp-training/mlvec_sw.slang:31-34), with every term a fused multiply-add;
 *     dW = dy (x) x, db = dy, dx = W^T dy (examples/mlp-training/mlp_sw.slang:28-58);
 *   - activations and their derivatives: source/standard-modules/neural/activations.slang:8-228 and
 *     the max tie rule of source/slang/diff.meta.slang:2268-2273;
 *   - Adam with eps inside the square root, NaN skip and inf clamp
 *     (examples/mlp-training/adam.slang:21-37, examples/mlp-training/kernels.slang:30-41);
 *   - loss word: float bits of the largest per-sample loss, combined with an unsigned max
 *     (examples/mlp-training/kernels.slang:22-27).
 *
 * Two flavours live here:
 *   (1) mlp_oracle_example_*: the literal 4->16->4 half-precision example with all of its quirks
 *       (leaky slope 0.001 forward but 0.01 backward, half accumulation from the bias, half Adam).
 *   (2) mlp_oracle_*: the same step parametrised by MlpConfig (widths, storage type, activation,
 *       loss, Adam constants) with a choice of accumulation type for the layer sums.
 *
 * Pinning: the per-operation behaviour is checked against the known answers of the reference's own
 * tests (tests/neural/basic-ilayer-ffn-{forward,backward}-test.slang,
 * tests/neural/fflayer-wavetangled-vector-test.slang, tests/neural/activation-functions-test.slang,
 * tests/cooperative-vector/{matrix-mul-bias,outer-product,reduce-sum-accumulate}.slang) in
 * tests/test_oracle_kat.py.  No reference test pins a multi-step trajectory or Adam: for those the
 * parity is unpinned by the reference and defined by this file.
 */
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "../include/slang_b200_mlp_config.h"

namespace {

// ---------------------------------------------------------------------------------------------
// Storage-type rounding (round to nearest even), done on the bit patterns so that the result does
// not depend on compiler flags.
// ---------------------------------------------------------------------------------------------
inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

inline uint16_t f32_to_bf16_bits(float f)
{
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x0040u);  // quiet NaN
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return uint16_t(u >> 16);
}
inline float bf16_bits_to_f32(uint16_t h) { return u2f(uint32_t(h) << 16); }

inline uint16_t f32_to_f16_bits(float f)
{
    _Float16 h = (_Float16)f;  // IEEE round-to-nearest-even conversion
    uint16_t b; std::memcpy(&b, &h, 2); return b;
}
inline float f16_bits_to_f32(uint16_t b)
{
    _Float16 h; std::memcpy(&h, &b, 2); return (float)h;
}

inline float round_to(int dtype, float v)
{
    switch (dtype) {
    case MLP_F16: return f16_bits_to_f32(f32_to_f16_bits(v));
    case MLP_BF16: return bf16_bits_to_f32(f32_to_bf16_bits(v));
    default: return v;
    }
}
inline int dtype_size(int dtype) { return dtype == MLP_F32 ? 4 : 2; }

inline float load_as_f32(int dtype, const void* base, int64_t idx)
{
    switch (dtype) {
    case MLP_F16: return f16_bits_to_f32(((const uint16_t*)base)[idx]);
    case MLP_BF16: return bf16_bits_to_f32(((const uint16_t*)base)[idx]);
    default: return ((const float*)base)[idx];
    }
}
inline void store_from_f32(int dtype, void* base, int64_t idx, float v)
{
    switch (dtype) {
    case MLP_F16: ((uint16_t*)base)[idx] = f32_to_f16_bits(v); break;
    case MLP_BF16: ((uint16_t*)base)[idx] = f32_to_bf16_bits(v); break;
    default: ((float*)base)[idx] = v; break;
    }
}

// ---------------------------------------------------------------------------------------------
// Activations (value and derivative with respect to the pre-activation x).
// ---------------------------------------------------------------------------------------------
const float kSqrt2OverPi = 0.7978845608028654f;
const float kGeluC = 0.044715f;

inline float act_value(int act, float alpha, float x)
{
    switch (act) {
    case MLP_ACT_RELU: return x > 0.0f ? x : 0.0f;
    case MLP_ACT_LEAKY_RELU: return x < 0.0f ? alpha * x : x;
    case MLP_ACT_LEAKY_MAX: { float y = x * alpha; return x > y ? x : y; }
    case MLP_ACT_SIGMOID: {
        float ex = std::exp(x >= 0.0f ? -x : x);
        return x >= 0.0f ? 1.0f / (1.0f + ex) : ex / (1.0f + ex);
    }
    case MLP_ACT_TANH: return std::tanh(x);
    case MLP_ACT_EXP: return std::exp(x);
    case MLP_ACT_SINE: return std::sin(x);
    case MLP_ACT_SILU: {
        float ex = std::exp(x >= 0.0f ? -x : x);
        return x >= 0.0f ? x / (1.0f + ex) : x * ex / (1.0f + ex);
    }
    case MLP_ACT_QUICK_GELU: {
        float sx = 1.702f * x;
        float ex = std::exp(sx >= 0.0f ? -sx : sx);
        return sx >= 0.0f ? x / (1.0f + ex) : x * ex / (1.0f + ex);
    }
    case MLP_ACT_GELU_TANH: {
        float u = kSqrt2OverPi * (x + kGeluC * x * x * x);
        return 0.5f * x * (1.0f + std::tanh(u));
    }
    default: return x;
    }
}

inline float sigmoidf(float x)
{
    float ex = std::exp(x >= 0.0f ? -x : x);
    return x >= 0.0f ? 1.0f / (1.0f + ex) : ex / (1.0f + ex);
}

inline float act_deriv(int act, float alpha, float x)
{
    switch (act) {
    case MLP_ACT_RELU: return x > 0.0f ? 1.0f : (x == 0.0f ? 0.5f : 0.0f);
    case MLP_ACT_LEAKY_RELU: return x < 0.0f ? alpha : 1.0f;
    case MLP_ACT_LEAKY_MAX: {
        // d max(x, alpha x): the larger side gets the gradient, a tie splits it in half.
        float y = x * alpha;
        if (x > y) return 1.0f;
        if (x < y) return alpha;
        return 0.5f * (1.0f + alpha);
    }
    case MLP_ACT_SIGMOID: { float s = sigmoidf(x); return s * (1.0f - s); }
    case MLP_ACT_TANH: { float t = std::tanh(x); return 1.0f - t * t; }
    case MLP_ACT_EXP: return std::exp(x);
    case MLP_ACT_SINE: return std::cos(x);
    case MLP_ACT_SILU: { float s = sigmoidf(x); return s * (1.0f + x * (1.0f - s)); }
    case MLP_ACT_QUICK_GELU: {
        float s = sigmoidf(1.702f * x);
        return s * (1.0f + 1.702f * x * (1.0f - s));
    }
    case MLP_ACT_GELU_TANH: {
        float x2 = x * x;
        float u = kSqrt2OverPi * (x + kGeluC * x * x2);
        float t = std::tanh(u);
        float du = kSqrt2OverPi * (1.0f + 3.0f * kGeluC * x2);
        return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
    }
    default: return 1.0f;
    }
}

// ---------------------------------------------------------------------------------------------
// Parameter layout: segment 1 is W0|b0|W1|b1|..., every sub-allocation rounded up to 64 bytes of
// the storage type (examples/mlp-training/mlp-training.cpp:217-250).  Offsets are in elements; the
// gradient segment and the Adam states use the same element offsets.
// ---------------------------------------------------------------------------------------------
struct Layout {
    int64_t w[MLP_MAX_LAYERS];
    int64_t b[MLP_MAX_LAYERS];
    int64_t total;
};

Layout make_layout(const MlpConfig& c)
{
    Layout L{};
    const int64_t align = 64 / dtype_size(c.dtype);
    int64_t off = 0;
    for (int l = 0; l < c.n_layers; ++l) {
        int64_t nw = int64_t(c.dims[l]) * c.dims[l + 1];
        L.w[l] = off; off += (nw + align - 1) / align * align;
        L.b[l] = off; off += (int64_t(c.dims[l + 1]) + align - 1) / align * align;
    }
    L.total = off;
    return L;
}

bool config_ok(const MlpConfig* c)
{
    if (!c || c->n_layers < 1 || c->n_layers > MLP_MAX_LAYERS) return false;
    for (int l = 0; l <= c->n_layers; ++l)
        if (c->dims[l] < 1 || c->dims[l] > 1024) return false;
    if (c->encoding == MLP_ENC_FREQ2D && (c->dims[0] != 32 || c->input_width != 2)) return false;
    if (c->encoding == MLP_ENC_NONE && c->input_width != c->dims[0]) return false;
    return true;
}

// Accumulating a * b into acc in the chosen accumulation type.
//   acc_mode 0: float; a rounded product then a rounded add (MLP_SUM_NEURAL) or one fused
//               multiply-add per term (MLP_SUM_BIAS_FIRST_FUSED)
//   acc_mode 1: double
//   acc_mode 2: the storage type (the literal CoopVec fallback, hlsl.meta.slang:32858-32869)
// This file is compiled with -ffp-contract=off: `acc + a * b` below is two roundings.
template <typename Acc> struct AccOps;
template <> struct AccOps<float> {
    static inline float mac(float acc, float a, float b, bool fused)
    {
        if (fused) return std::fmaf(a, b, acc);
        const float prod = a * b;
        return acc + prod;
    }
};
template <> struct AccOps<double> {
    static inline double mac(double acc, float a, float b, bool) { return acc + double(a) * double(b); }
};

const float kPi = 3.14159265358979323846f;

// The type a product reads its operands in: the storage type, or MlpConfig.operand_dtype for fp32 storage with
// 16-bit tensor-core operands (the neural module's T = float: source/standard-modules/neural/
// mma-tiled-cuda.slang:104-118 converts both matrix operands to half whatever the element type is).
inline int operand_type(const MlpConfig& c) { return c.operand_dtype ? c.operand_dtype : c.dtype; }
inline float round_op(const MlpConfig& c, float v) { return round_to(operand_type(c), v); }


void encode_input(const MlpConfig& c, const void* inputs, int64_t s, float* a0)
{
    if (c.encoding == MLP_ENC_FREQ2D) {
        for (int u = 0; u < 2; ++u) {
            float v = load_as_f32(c.input_dtype, inputs, s * 2 + u);
            for (int k = 0; k < 8; ++k) {
                float arg = std::ldexp(kPi, k) * v;
                a0[u * 16 + k * 2 + 0] = round_op(c, std::sin(arg));
                a0[u * 16 + k * 2 + 1] = round_op(c, std::cos(arg));
            }
        }
    } else {
        for (int i = 0; i < c.dims[0]; ++i)
            a0[i] = round_op(c, load_as_f32(c.input_dtype, inputs, s * c.dims[0] + i));
    }
}

// The parameters widened to float once per call (exact: every storage type embeds in float), so
// that the inner loops do not convert on every multiply.
struct FloatParams {
    std::vector<float> v;
    FloatParams(const MlpConfig& c, const Layout& L, const void* params) : v(size_t(L.total))
    {
        for (int64_t i = 0; i < L.total; ++i) v[size_t(i)] = load_as_f32(c.dtype, params, i);
        if (c.operand_dtype) {
            // weights as the products read them; biases keep the storage type
            for (int l = 0; l < c.n_layers; ++l)
                for (int64_t i = 0; i < int64_t(c.dims[l]) * c.dims[l + 1]; ++i)
                    v[size_t(L.w[l] + i)] = round_op(c, v[size_t(L.w[l] + i)]);
        }
    }
};

struct Scratch {
    std::vector<float> a[MLP_MAX_LAYERS + 1];  // a[l]: vector entering layer l (storage-rounded)
    std::vector<float> z[MLP_MAX_LAYERS];      // z[l]: pre-activation of layer l (storage-rounded)
    std::vector<float> dz, da;
    explicit Scratch(const MlpConfig& c)
    {
        int mx = 0;
        for (int l = 0; l <= c.n_layers; ++l) { a[l].assign(c.dims[l], 0.f); mx = std::max(mx, c.dims[l]); }
        for (int l = 0; l < c.n_layers; ++l) z[l].assign(c.dims[l + 1], 0.f);
        dz.assign(mx, 0.f); da.assign(mx, 0.f);
    }
};

// Forward pass of one sample.  On return sc.a[n_layers] holds the network output in fp32
// (output activation applied, not rounded to the storage type).
template <typename Acc>
void forward_sample(const MlpConfig& c, const Layout& L, const float* params, const void* inputs, int64_t s,
                    Scratch& sc, int acc_mode)
{
    encode_input(c, inputs, s, sc.a[0].data());
    const bool bias_first = c.sum_order == MLP_SUM_BIAS_FIRST_FUSED;
    for (int l = 0; l < c.n_layers; ++l) {
        const int in = c.dims[l], out = c.dims[l + 1];
        const bool last = (l == c.n_layers - 1);
        for (int j = 0; j < out; ++j) {
            float bias = params[L.b[l] + j];
            const float* wrow = params + L.w[l] + int64_t(j) * in;
            const float* ain = sc.a[l].data();
            float zf;
            if (acc_mode == 2) {
                float r = bias_first ? bias : 0.0f;
                for (int i = 0; i < in; ++i) {
                    float prod = round_to(c.dtype, wrow[i] * ain[i]);
                    r = round_to(c.dtype, r + prod);
                }
                zf = bias_first ? r : round_to(c.dtype, r + bias);
            } else {
                Acc r = bias_first ? Acc(bias) : Acc(0);
                for (int i = 0; i < in; ++i) r = AccOps<Acc>::mac(r, wrow[i], ain[i], bias_first);
                if (!bias_first) r = r + Acc(bias);
                zf = float(r);
            }
            float zs = round_to(c.dtype, zf);
            sc.z[l][j] = zs;
            if (last) sc.a[l + 1][j] = act_value(c.output_act, c.act_alpha, zs);
            else sc.a[l + 1][j] = round_op(c, act_value(c.hidden_act, c.act_alpha, zs));
        }
    }
}

template <typename Acc>
float learn_sample(const MlpConfig& c, const Layout& L, const float* params, float* grads, const void* inputs,
                   const void* targets, int64_t s, Scratch& sc, int acc_mode, float* input_grads = nullptr)
{
    forward_sample<Acc>(c, L, params, inputs, s, sc, acc_mode);
    const int nl = c.n_layers;
    const int od = c.dims[nl];
    // Loss and its gradient with respect to the last pre-activation.
    float loss = 0.0f;
    const bool fused = c.sum_order == MLP_SUM_BIAS_FIRST_FUSED;
    const float scale = (c.loss == MLP_LOSS_MSE_MEAN) ? 1.0f / float(od) : 1.0f;
    for (int j = 0; j < od; ++j) {
        float t = load_as_f32(c.target_dtype, targets, s * od + j);
        float diff = sc.a[nl][j] - t;
        loss = std::fmaf(diff * scale, diff, loss);
        float dout = 2.0f * scale * diff;
        float d = act_deriv(c.output_act, c.act_alpha, sc.z[nl - 1][j]);
        sc.dz[j] = round_op(c, dout * d);
    }
    for (int l = nl - 1; l >= 0; --l) {
        const int in = c.dims[l], out = c.dims[l + 1];
        // dW += dz (x) a, db += dz : plain load-add-store in ascending sample order.
        for (int j = 0; j < out; ++j) {
            const float g = sc.dz[j];
            float* gw = grads + L.w[l] + int64_t(j) * in;
            if (fused) {
                for (int i = 0; i < in; ++i) gw[i] = std::fmaf(g, sc.a[l][i], gw[i]);
            } else {
                for (int i = 0; i < in; ++i) {
                    const float prod = sc.a[l][i] * g;  // T prod = x * dy; then the add
                    gw[i] = gw[i] + prod;
                }
            }
            grads[L.b[l] + j] += g;
        }
        if (l == 0) {
            // The example's inputs are no_diff, so this gradient is dead there; an encoder in front of the
            // network needs it: dx = W_0^T dz_0 (same accumulation as the hidden layers), rounded to the
            // storage type, one row of dims[0] floats per sample.
            if (input_grads) {
                for (int i = 0; i < in; ++i) {
                    Acc r = Acc(0);
                    const float* wcol = params + L.w[0] + i;
                    for (int j = 0; j < out; ++j) r = AccOps<Acc>::mac(r, wcol[int64_t(j) * in], sc.dz[j], fused);
                    input_grads[s * in + i] = round_to(c.dtype, float(r));
                }
            }
            break;
        }
        // da = W^T dz, then through the previous activation.
        for (int i = 0; i < in; ++i) {
            float v;
            if (acc_mode == 2) {
                float r = 0.0f;
                for (int j = 0; j < out; ++j) {
                    float prod = round_to(c.dtype, params[L.w[l] + int64_t(j) * in + i] * sc.dz[j]);
                    r = round_to(c.dtype, r + prod);
                }
                v = r;
            } else {
                Acc r = Acc(0);
                const float* wcol = params + L.w[l] + i;
                for (int j = 0; j < out; ++j) r = AccOps<Acc>::mac(r, wcol[int64_t(j) * in], sc.dz[j], fused);
                v = float(r);
            }
            float d = round_op(c, act_deriv(c.hidden_act, c.act_alpha, sc.z[l - 1][i]));
            sc.da[i] = round_op(c, v * d);
        }
        std::swap(sc.dz, sc.da);
    }
    return loss;
}

template <typename Acc>
void learn_range(const MlpConfig& c, const Layout& L, const float* params, float* grads, const void* inputs,
                 const void* targets, int64_t s0, int64_t s1, int acc_mode, float* max_loss, double* sum_loss,
                 float* input_grads = nullptr)
{
    Scratch sc(c);
    float mx = 0.0f;
    double sum = 0.0;
    for (int64_t s = s0; s < s1; ++s) {
        float l = learn_sample<Acc>(c, L, params, grads, inputs, targets, s, sc, acc_mode, input_grads);
        if (l > mx) mx = l;
        sum += double(l);
    }
    *max_loss = mx;
    *sum_loss = sum;
}

// Integer power by repeated squaring in float: the same sequence of correctly rounded multiplies
// on every machine (the reference calls pow(beta, NFloat(iteration)), adam.slang:33-34).
inline float pow_int(float base, int32_t e)
{
    float r = 1.0f, b = base;
    while (e > 0) {
        if (e & 1) r = r * b;
        b = b * b;
        e >>= 1;
    }
    return r;
}

}  // namespace

extern "C" {

// Element offsets of each layer's weights and biases and the padded total.
int mlp_oracle_param_layout(const MlpConfig* c, int64_t* w_off, int64_t* b_off, int64_t* total)
{
    if (!config_ok(c)) return -1;
    Layout L = make_layout(*c);
    for (int l = 0; l < c->n_layers; ++l) { w_off[l] = L.w[l]; b_off[l] = L.b[l]; }
    *total = L.total;
    return 0;
}

// out: [count][dims[n_layers]] fp32 network outputs (output activation applied).
int mlp_oracle_forward(const MlpConfig* c, const void* params, const void* inputs, int64_t count, float* out,
                       int acc_mode)
{
    if (!config_ok(c)) return -1;
    Layout L = make_layout(*c);
    Scratch sc(*c);
    FloatParams fp(*c, L, params);
    const int od = c->dims[c->n_layers];
    for (int64_t s = 0; s < count; ++s) {
        if (acc_mode == 1) forward_sample<double>(*c, L, fp.v.data(), inputs, s, sc, acc_mode);
        else forward_sample<float>(*c, L, fp.v.data(), inputs, s, sc, acc_mode);
        std::memcpy(out + s * od, sc.a[c->n_layers].data(), sizeof(float) * od);
    }
    return 0;
}

// The learnGradient step: grads (fp32, padded layout) += sum over samples; loss_words[0] is combined
// by unsigned max with the float bits of the largest per-sample loss, loss_words[1] receives the
// float bits of (previous value + sum of per-sample losses).
// n_threads <= 1: the literal CPU-target order (one thread, ascending samples).
// n_threads  > 1: disjoint contiguous sample ranges, one private gradient copy per thread, copies
//                 added to grads in thread order (the documented group-range ABI, docs/cpu-target.md:404).
int mlp_oracle_learn_gradient(const MlpConfig* c, const void* params, float* grads, const void* inputs,
                              const void* targets, int64_t count, uint32_t* loss_words, int acc_mode, int n_threads)
{
    if (!config_ok(c)) return -1;
    Layout L = make_layout(*c);
    FloatParams fpar(*c, L, params);
    const float* pf = fpar.v.data();
    float mx = 0.0f;
    double sum = 0.0;
    if (n_threads <= 1) {
        if (acc_mode == 1) learn_range<double>(*c, L, pf, grads, inputs, targets, 0, count, acc_mode, &mx, &sum);
        else learn_range<float>(*c, L, pf, grads, inputs, targets, 0, count, acc_mode, &mx, &sum);
    } else {
        std::vector<std::vector<float>> priv(n_threads, std::vector<float>(size_t(L.total), 0.0f));
        std::vector<float> mxs(n_threads, 0.0f);
        std::vector<double> sums(n_threads, 0.0);
        std::vector<std::thread> th;
        for (int t = 0; t < n_threads; ++t) {
            int64_t s0 = count * t / n_threads, s1 = count * (t + 1) / n_threads;
            th.emplace_back([&, t, s0, s1]() {
                if (acc_mode == 1)
                    learn_range<double>(*c, L, pf, priv[t].data(), inputs, targets, s0, s1, acc_mode, &mxs[t], &sums[t]);
                else
                    learn_range<float>(*c, L, pf, priv[t].data(), inputs, targets, s0, s1, acc_mode, &mxs[t], &sums[t]);
            });
        }
        for (auto& t : th) t.join();
        for (int t = 0; t < n_threads; ++t) {
            for (int64_t i = 0; i < L.total; ++i) grads[i] += priv[t][i];
            mx = std::max(mx, mxs[t]);
            sum += sums[t];
        }
    }
    if (loss_words) {
        uint32_t bits = f2u(mx);
        if (bits > loss_words[0]) loss_words[0] = bits;
        loss_words[1] = f2u(u2f(loss_words[1]) + float(sum));
    }
    return 0;
}

// learnGradient that also returns the gradient with respect to the (unencoded) inputs: input_grads is
// [count][dims[0]] fp32.  One thread, fp32 fused multiply-add accumulation.
int mlp_oracle_learn_gradient_inputs(const MlpConfig* c, const void* params, float* grads, const void* inputs,
                                     const void* targets, int64_t count, uint32_t* loss_words, float* input_grads)
{
    if (!config_ok(c) || c->encoding != MLP_ENC_NONE) return -1;
    Layout L = make_layout(*c);
    FloatParams fpar(*c, L, params);
    float mx = 0.0f;
    double sum = 0.0;
    learn_range<float>(*c, L, fpar.v.data(), grads, inputs, targets, 0, count, 0, &mx, &sum, input_grads);
    if (loss_words) {
        uint32_t bits = f2u(mx);
        if (bits > loss_words[0]) loss_words[0] = bits;
        loss_words[1] = f2u(u2f(loss_words[1]) + float(sum));
    }
    return 0;
}

// The adjustParameters step over `count` elements of the padded layout.
int mlp_oracle_adjust_parameters(const MlpConfig* c, MlpAdamState* states, void* params, float* grads, int64_t count)
{
    if (!config_ok(c)) return -1;
    for (int64_t i = 0; i < count; ++i) {
        float g = grads[i];
        if (std::isnan(g)) { grads[i] = 0.0f; continue; }
        MlpAdamState& st = states[i];
        st.iteration++;
        if (std::isinf(g)) g = g > 0 ? 10000.0f : -10000.0f;
        st.mean = c->beta1 * st.mean + (1.0f - c->beta1) * g;
        st.variance = c->beta2 * st.variance + ((1.0f - c->beta2) * g) * g;
        float mean_hat = st.mean / (1.0f - pow_int(c->beta1, st.iteration));
        float var_hat = st.variance / (1.0f - pow_int(c->beta2, st.iteration));
        float p = c->adam_master ? st.master : load_as_f32(c->dtype, params, i);
        float denom = std::sqrt(std::max(0.0f, var_hat) + c->eps);
        p = p - (c->lr * mean_hat) / denom;
        st.master = p;
        store_from_f32(c->dtype, params, i, p);
        grads[i] = 0.0f;
    }
    return 0;
}

// Storage-type conversion helpers for building test vectors.
void mlp_oracle_convert_from_f32(int dtype, const float* src, void* dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) store_from_f32(dtype, dst, i, src[i]);
}
void mlp_oracle_convert_to_f32(int dtype, const void* src, float* dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) dst[i] = load_as_f32(dtype, src, i);
}
float mlp_oracle_activation(int act, float alpha, float x) { return act_value(act, alpha, x); }
float mlp_oracle_activation_deriv(int act, float alpha, float x) { return act_deriv(act, alpha, x); }

// ---------------------------------------------------------------------------------------------
// The literal example: 4 -> 16 -> 4, everything in half (examples/mlp-training/*.slang).
// ---------------------------------------------------------------------------------------------
}  // extern "C"

typedef _Float16 hf;

static inline hf ld_h(uint64_t addr, int i) { hf v; std::memcpy(&v, (const char*)addr + 2 * i, 2); return v; }
static inline void add_h(uint64_t addr, int i, hf v)
{
    // InterlockedAddF16Emulated on a sequential machine: load, add in half, store.
    hf cur = ld_h(addr, i);
    cur = cur + v;
    std::memcpy((char*)addr + 2 * i, &cur, 2);
}

template <int In, int Out>
static void ex_layer_eval(const MlpLayerPointers& lp, const hf* x, hf* y)
{
    for (int i = 0; i < Out; ++i) {
        hf r = ld_h(lp.biases, i);
        for (int j = 0; j < In; ++j) r += ld_h(lp.weights, i * In + j) * x[j];
        y[i] = r;
    }
    for (int i = 0; i < Out; ++i)
        if (y[i] < (hf)0.0f) y[i] *= (hf)0.001f;  // mlp_sw.slang:22-24
}

template <int In, int Out>
static void ex_layer_bwd(const MlpLayerPointers& lp, const hf* x, hf* g /*[Out], modified*/, hf* dx /*[In]*/)
{
    hf fwd[Out];
    ex_layer_eval<In, Out>(lp, x, fwd);
    for (int i = 0; i < Out; ++i)
        if (fwd[i] < (hf)0.0f) g[i] *= (hf)0.01f;  // mlp_sw.slang:35-39 (not the forward slope)
    for (int i = 0; i < Out; ++i)
        for (int j = 0; j < In; ++j) add_h(lp.weightsGrad, i * In + j, g[i] * x[j]);
    for (int i = 0; i < Out; ++i) add_h(lp.biasesGrad, i, g[i]);
    for (int i = 0; i < In; ++i) {
        hf r = (hf)0.0f;
        for (int j = 0; j < Out; ++j) r += ld_h(lp.weights, j * In + i) * g[j];
        dx[i] = r;
    }
}

// The cooperative-vector flavour of the example (examples/mlp-training-coopvec/fflayer.slang:16-66):
// matrix-vector sums start from zero and the bias is added afterwards (source/slang/hlsl.meta.slang:
// 32858-32912 and the bias loop after it); activation max(o, o * 0.001h).
template <int In, int Out>
static void cv_layer_sums(const MlpLayerPointers& lp, const hf* x, hf* o)
{
    for (int i = 0; i < Out; ++i) {
        hf r = (hf)0.0f;
        for (int j = 0; j < In; ++j) r += ld_h(lp.weights, i * In + j) * x[j];
        o[i] = r + ld_h(lp.biases, i);
    }
}

template <int N>
static void cv_activation(const hf* o, hf* y)
{
    for (int i = 0; i < N; ++i) {
        const hf scaled = o[i] * (hf)0.001f;
        y[i] = o[i] > scaled ? o[i] : (o[i] < scaled ? scaled : o[i]);
    }
}

// Reverse pass of one layer: max's derivative gives the whole gradient to the larger argument and half
// to each at a tie (source/slang/diff.meta.slang:2268-2273); the second argument is o * 0.001h.  The
// weight gradient goes to a 16x16 tile (the training-optimal layout of this library for matrices up to
// 16x16: element (i, j) at i * 16 + j) by plain load-add-store (hlsl.meta.slang:33261-33315), the bias
// gradient to its row-major slot (hlsl.meta.slang:33344-33351), dx = W^T g from zero.
template <int In, int Out>
static void cv_layer_bwd(const MlpLayerPointers& lp, const hf* x, const hf* o, hf* g, hf* dx)
{
    for (int i = 0; i < Out; ++i) {
        const hf scaled = o[i] * (hf)0.001f;
        if (o[i] > scaled) { /* first argument takes it all */ }
        else if (o[i] < scaled) g[i] = g[i] * (hf)0.001f;
        else { const hf h = (hf)0.5f * g[i]; g[i] = h + h * (hf)0.001f; }
    }
    for (int i = 0; i < Out; ++i)
        for (int j = 0; j < In; ++j) add_h(lp.weightsGrad, i * 16 + j, g[i] * x[j]);
    for (int i = 0; i < Out; ++i) add_h(lp.biasesGrad, i, g[i]);
    for (int i = 0; i < In; ++i) {
        hf r = (hf)0.0f;
        for (int j = 0; j < Out; ++j) r += ld_h(lp.weights, j * In + i) * g[j];
        dx[i] = r;
    }
}

static void ex_groundtruth(hf x, hf y, hf* gt)
{
    gt[0] = (x + y) / ((hf)1.0f + y * y);
    gt[1] = (hf)2.0f * x + y;
    gt[2] = (hf)0.5f * x * x + (hf)1.2f * y;
    gt[3] = x + (hf)0.5f * y * y;
}

extern "C" {

// learnGradient of the example over `count` samples; network points at two MlpLayerPointers with
// host addresses; inputs is count float2.
static void ex_learn_thread(uint32_t tid, const MlpLayerPointers* network, uint32_t* loss_word, const float* inputs,
                            uint32_t count)
{
    if (tid >= count) return;
    hf x = (hf)inputs[2 * tid], y = (hf)inputs[2 * tid + 1];
    hf enc[4] = {x, y, x * x, y * y};
    hf h1[16], out[4], gt[4], diff[4];
    ex_layer_eval<4, 16>(network[0], enc, h1);
    ex_layer_eval<16, 4>(network[1], h1, out);
    ex_groundtruth(x, y, gt);
    for (int k = 0; k < 4; ++k) diff[k] = out[k] - gt[k];
    // d dot(diff, diff) with dOut = 1: each factor contributes diff * dOut (diff.meta.slang:1608-1621).
    hf g2[4];
    for (int k = 0; k < 4; ++k) g2[k] = diff[k] * (hf)1.0f + diff[k] * (hf)1.0f;
    hf g1[16], dead[4];
    ex_layer_bwd<16, 4>(network[1], h1, g2, g1);
    ex_layer_bwd<4, 16>(network[0], enc, g1, dead);
    hf l = (hf)0.0f;
    for (int k = 0; k < 4; ++k) l += diff[k] * diff[k];
    uint32_t bits = f2u((float)l);
    if (bits > *loss_word) *loss_word = bits;
}

int mlp_oracle_example_learn_gradient(const MlpLayerPointers* network, uint32_t* loss_word, const float* inputs,
                                      uint32_t count)
{
    for (uint32_t tid = 0; tid < count; ++tid) ex_learn_thread(tid, network, loss_word, inputs, count);
    return 0;
}

// learnGradient of the cooperative-vector example (examples/mlp-training-coopvec/kernels.slang:7-27).
int mlp_oracle_example_coopvec_learn_gradient(const MlpLayerPointers* network, uint32_t* loss_word, const float* inputs,
                                              uint32_t count)
{
    for (uint32_t tid = 0; tid < count; ++tid) {
        hf x = (hf)inputs[2 * tid], y = (hf)inputs[2 * tid + 1];
        hf enc[4] = {x, y, x * x, y * y};
        hf o1[16], h1[16], o2[4], out[4], gt[4], diff[4];
        cv_layer_sums<4, 16>(network[0], enc, o1);
        cv_activation<16>(o1, h1);
        cv_layer_sums<16, 4>(network[1], h1, o2);
        cv_activation<4>(o2, out);
        ex_groundtruth(x, y, gt);
        for (int k = 0; k < 4; ++k) diff[k] = out[k] - gt[k];
        hf g2[4];
        for (int k = 0; k < 4; ++k) g2[k] = diff[k] * (hf)1.0f + diff[k] * (hf)1.0f;
        hf g1[16], dead[4];
        cv_layer_bwd<16, 4>(network[1], h1, o2, g2, g1);
        cv_layer_bwd<4, 16>(network[0], enc, o1, g1, dead);
        hf l = (hf)0.0f;
        for (int k = 0; k < 4; ++k) l += diff[k] * diff[k];
        uint32_t bits = f2u((float)l);
        if (bits > *loss_word) *loss_word = bits;
    }
    return 0;
}

static void ex_adjust_thread(uint32_t i, MlpExampleAdamState* states, uint16_t* params, uint16_t* grads, uint32_t count)
{
    if (i >= count) return;
    const hf beta1 = (hf)0.9f, beta2 = (hf)0.999f, eps = (hf)1e-7f, lr = (hf)0.01f;
    hf g; std::memcpy(&g, &grads[i], 2);
    if (g != g) { grads[i] = 0; return; }
    hf p; std::memcpy(&p, &params[i], 2);
    hf m, v; std::memcpy(&m, &states[i].mean, 2); std::memcpy(&v, &states[i].variance, 2);
    states[i].iteration++;
    if (std::isinf((float)g)) g = g > (hf)0.0f ? (hf)10000.0f : (hf)-10000.0f;
    m = beta1 * m + ((hf)1.0f - beta1) * g;
    v = beta2 * v + ((hf)1.0f - beta2) * g * g;
    hf it = (hf)(float)states[i].iteration;
    hf mean_hat = m / ((hf)1.0f - (hf)std::pow((float)beta1, (float)it));
    hf var_hat = v / ((hf)1.0f - (hf)std::pow((float)beta2, (float)it));
    hf mx = var_hat > (hf)0.0f ? var_hat : (hf)0.0f;
    hf den = (hf)std::sqrt((float)(hf)(mx + eps));
    p -= lr * mean_hat / den;
    std::memcpy(&params[i], &p, 2);
    std::memcpy(&states[i].mean, &m, 2); std::memcpy(&states[i].variance, &v, 2);
    grads[i] = 0;
}

int mlp_oracle_example_adjust_parameters(MlpExampleAdamState* states, uint16_t* params, uint16_t* grads, uint32_t count)
{
    for (uint32_t i = 0; i < count; ++i) ex_adjust_thread(i, states, params, grads, count);
    return 0;
}

// ---------------------------------------------------------------------------------------------
// The two example kernels behind the calling convention of a compute entry point compiled for the
// CPU (docs/cpu-target.md:363-424, prelude/slang-cpp-types.h:1336-1358): per entry point three
// exported functions.  `name` runs the groups of [startGroupID, endGroupID), `name_Group` runs the one
// group startGroupID, `name_Thread` runs one thread; groups in ascending order and the 256 threads of
// a group in ascending order (source/slang/slang-emit-cpp.cpp:2210-2284).  entryPointParams is the
// packed uniform parameter struct (pointers at 0/8/16, count at 24, examples/mlp-training/
// mlp-training.cpp:55-69) holding host addresses; globalParams is unused.  The kernels are
// one-dimensional: the y and z ranges must be [0,1).
// ---------------------------------------------------------------------------------------------
struct OracleUint3 { uint32_t x, y, z; };
struct OracleComputeVaryingInput { OracleUint3 startGroupID, endGroupID; };
struct OracleComputeThreadVaryingInput { OracleUint3 groupID, groupThreadID; };
struct OracleEntryParams { uint64_t p0, p1, p2; uint32_t count; };

static const uint32_t kGroupThreads = 256;  // [numthreads(256,1,1)], examples/mlp-training/kernels.slang:7,29

static void learn_run_thread(uint32_t tid, const void* ep)
{
    OracleEntryParams a; std::memcpy(&a, ep, 28);
    ex_learn_thread(tid, (const MlpLayerPointers*)(uintptr_t)a.p0, (uint32_t*)(uintptr_t)a.p1, (const float*)(uintptr_t)a.p2, a.count);
}
static void adjust_run_thread(uint32_t tid, const void* ep)
{
    OracleEntryParams a; std::memcpy(&a, ep, 28);
    ex_adjust_thread(tid, (MlpExampleAdamState*)(uintptr_t)a.p0, (uint16_t*)(uintptr_t)a.p1, (uint16_t*)(uintptr_t)a.p2, a.count);
}

void learnGradient_Thread(OracleComputeThreadVaryingInput* v, void* entryPointParams, void*)
{
    learn_run_thread(v->groupID.x * kGroupThreads + v->groupThreadID.x, entryPointParams);
}
void learnGradient_Group(OracleComputeVaryingInput* v, void* entryPointParams, void*)
{
    for (uint32_t t = 0; t < kGroupThreads; ++t) learn_run_thread(v->startGroupID.x * kGroupThreads + t, entryPointParams);
}
void learnGradient(OracleComputeVaryingInput* v, void* entryPointParams, void*)
{
    for (uint32_t g = v->startGroupID.x; g < v->endGroupID.x; ++g)
        for (uint32_t t = 0; t < kGroupThreads; ++t) learn_run_thread(g * kGroupThreads + t, entryPointParams);
}
void adjustParameters_Thread(OracleComputeThreadVaryingInput* v, void* entryPointParams, void*)
{
    adjust_run_thread(v->groupID.x * kGroupThreads + v->groupThreadID.x, entryPointParams);
}
void adjustParameters_Group(OracleComputeVaryingInput* v, void* entryPointParams, void*)
{
    for (uint32_t t = 0; t < kGroupThreads; ++t) adjust_run_thread(v->startGroupID.x * kGroupThreads + t, entryPointParams);
}
void adjustParameters(OracleComputeVaryingInput* v, void* entryPointParams, void*)
{
    for (uint32_t g = v->startGroupID.x; g < v->endGroupID.x; ++g)
        for (uint32_t t = 0; t < kGroupThreads; ++t) adjust_run_thread(g * kGroupThreads + t, entryPointParams);
}

// The host's float -> half conversion that initialises the example's parameters
// (examples/mlp-training/mlp-training.cpp:314-339).  It is not IEEE round-to-nearest-even: the
// mantissa is cut to one bit more than half keeps and that extra bit is added back (round half up);
// magnitudes below 2^-24 flush to zero and anything at or above 2^16 becomes infinity.
uint16_t mlp_oracle_example_float_to_half(float val)
{
    const uint32_t bits = f2u(val);
    const uint16_t sign = uint16_t((bits >> 16) & 0x8000u);
    const uint32_t biased = (bits >> 23) & 0xffu;
    const uint32_t frac = bits & 0x007fffffu;
    if (biased < 103u) return sign;
    if (biased > 142u) return uint16_t(sign | 0x7c00u | uint16_t(biased == 255u && frac != 0u));
    const uint32_t top11 = frac >> 12;  // ten kept bits and the rounding bit
    if (biased < 113u) {
        // subnormal half: make the hidden one explicit, shift into place, add the bit shifted out last
        const uint32_t sig = top11 | 0x800u;
        return uint16_t(sign | ((sig >> (114u - biased)) + ((sig >> (113u - biased)) & 1u)));
    }
    return uint16_t((sign | ((biased - 112u) << 10) | (top11 >> 1)) + (top11 & 1u));
}

}  // extern "C"
