// A second plain statement of the LlamaForCausalLM forward pass, in C++ (double precision, whole
// sequences, no cache), written from the reference's formulas and not from the NumPy one
// (tests/plain_llama.py): the two must agree to 1e-9 on the tiny configurations, which is the
// check that neither misreads the reference.  Citations are DeanoC/SuperSonic file:line.
//
// Input (binary, little-endian), written by tests/test_plain_impl.py:
//   int64  vocab, hidden, inter, layers, n_q, n_kv, head_dim, tied, n_tokens, has_scaling
//   double eps, theta, factor, low_freq_factor, high_freq_factor, original_max_positions
//   int64  tokens[n_tokens]
//   double embed[vocab*hidden]; per layer: ln1[hidden], q[n_q*hd*hidden], k[n_kv*hd*hidden], v[...],
//          o[hidden*n_q*hd], ln2[hidden], gate[inter*hidden], up[inter*hidden], down[hidden*inter];
//          norm[hidden]; head[vocab*hidden] unless tied
// Output: double logits[n_tokens*vocab].
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <vector>

typedef std::vector<double> vec;

static bool read_all(FILE* f, void* p, size_t bytes) { return fread(p, 1, bytes, f) == bytes; }

// y[t, n] = sum_k x[t, k] w[n, k]   (weights are [out, in], HF layout: llama31_engine.rs:177-246)
static vec linear(const vec& x, const double* w, int T, int K, int N) {
    vec y((size_t)T * N, 0.0);
    for (int t = 0; t < T; ++t)
        for (int n = 0; n < N; ++n) {
            double s = 0.0;
            const double* xr = &x[(size_t)t * K];
            const double* wr = w + (size_t)n * K;
            for (int k = 0; k < K; ++k) s += xr[k] * wr[k];
            y[(size_t)t * N + n] = s;
        }
    return y;
}

// y = x * rsqrt(mean(x^2) + eps) * w, weight used as w (kernels/full_attention_cuda.cuh:2826-2873;
// rms_norm_add_unit_offset false: llama31_engine.rs:89)
static vec rms_norm(const vec& x, const double* w, int T, int H, double eps) {
    vec y(x.size());
    for (int t = 0; t < T; ++t) {
        double ss = 0.0;
        for (int c = 0; c < H; ++c) ss += x[(size_t)t * H + c] * x[(size_t)t * H + c];
        const double r = 1.0 / std::sqrt(ss / H + eps);
        for (int c = 0; c < H; ++c) y[(size_t)t * H + c] = x[(size_t)t * H + c] * r * w[c];
    }
    return y;
}

int main(int argc, char** argv) {
    if (argc != 3) { fprintf(stderr, "usage: plain_llama IN OUT\n"); return 2; }
    FILE* f = fopen(argv[1], "rb");
    if (!f) { perror("open input"); return 1; }
    int64_t hdr[10];
    double par[6];
    if (!read_all(f, hdr, sizeof hdr) || !read_all(f, par, sizeof par)) { fprintf(stderr, "short header\n"); return 1; }
    const int V = (int)hdr[0], H = (int)hdr[1], I = (int)hdr[2], L = (int)hdr[3], nq = (int)hdr[4], nkv = (int)hdr[5],
              hd = (int)hdr[6], tied = (int)hdr[7], T = (int)hdr[8], scaled = (int)hdr[9];
    const double eps = par[0], theta = par[1], factor = par[2], low = par[3], high = par[4], old_ctx = par[5];
    std::vector<int64_t> tokens(T);
    if (!read_all(f, tokens.data(), sizeof(int64_t) * T)) { fprintf(stderr, "short tokens\n"); return 1; }
    auto read_vec = [&](size_t n) { vec v(n); if (!read_all(f, v.data(), n * sizeof(double))) { fprintf(stderr, "short weights\n"); exit(1); } return v; };
    const vec embed = read_vec((size_t)V * H);

    // llama3-scaled inverse frequencies (llama31_engine.rs:115-145) and angle = position * frequency (147-157)
    const double pi = std::acos(-1.0);
    vec inv(hd / 2);
    for (int i = 0; i < hd / 2; ++i) {
        const double base = 1.0 / std::pow(theta, 2.0 * i / hd);
        double fr = base;
        if (scaled) {
            const double wavelen = 2.0 * pi / base, low_wavelen = old_ctx / low, high_wavelen = old_ctx / high;
            if (wavelen > low_wavelen) fr = base / factor;
            else if (wavelen < high_wavelen) fr = base;
            else {
                const double smooth = (old_ctx / wavelen - low) / (high - low);
                fr = (1.0 - smooth) * base / factor + smooth * base;
            }
        }
        inv[i] = fr;
    }
    // half-split pairs (i, i + hd/2): kernels/prefill_helpers_cuda.cuh:80-111
    auto rope = [&](vec& x, int heads) {
        for (int t = 0; t < T; ++t)
            for (int h = 0; h < heads; ++h) {
                double* r = &x[((size_t)t * heads + h) * hd];
                for (int i = 0; i < hd / 2; ++i) {
                    const double a = t * inv[i], c = std::cos(a), s = std::sin(a);
                    const double x0 = r[i], x1 = r[i + hd / 2];
                    r[i] = x0 * c - x1 * s;
                    r[i + hd / 2] = x0 * s + x1 * c;
                }
            }
    };

    vec h((size_t)T * H);                                       // h[t] = E[id_t] (full_attention_cuda.cuh:2012-2034)
    for (int t = 0; t < T; ++t)
        for (int c = 0; c < H; ++c) h[(size_t)t * H + c] = embed[(size_t)tokens[t] * H + c];
    const double scale = 1.0 / std::sqrt((double)hd);           // prefill_engine.rs:2200
    const int group = nq / nkv;
    for (int l = 0; l < L; ++l) {
        const vec ln1 = read_vec(H), wq = read_vec((size_t)nq * hd * H), wk = read_vec((size_t)nkv * hd * H),
                  wv = read_vec((size_t)nkv * hd * H), wo = read_vec((size_t)H * nq * hd), ln2 = read_vec(H),
                  wg = read_vec((size_t)I * H), wu = read_vec((size_t)I * H), wd = read_vec((size_t)H * I);
        // pre-norm residual block (prefill_engine.rs:1116-1222)
        const vec x = rms_norm(h, ln1.data(), T, H, eps);
        vec q = linear(x, wq.data(), T, H, nq * hd), k = linear(x, wk.data(), T, H, nkv * hd);
        const vec v = linear(x, wv.data(), T, H, nkv * hd);
        rope(q, nq);
        rope(k, nkv);
        // causal GQA attention, query head g reads kv head g / (nq / nkv), max-subtracted softmax
        // (full_attention_cuda.cuh:360-474)
        vec a((size_t)T * nq * hd, 0.0);
        vec p(T);
        for (int g = 0; g < nq; ++g) {
            const int kvh = g / group;
            for (int t = 0; t < T; ++t) {
                double m = -INFINITY;
                for (int j = 0; j <= t; ++j) {
                    double s = 0.0;
                    for (int d = 0; d < hd; ++d) s += q[((size_t)t * nq + g) * hd + d] * k[((size_t)j * nkv + kvh) * hd + d];
                    p[j] = s * scale;
                    if (p[j] > m) m = p[j];
                }
                double denom = 0.0;
                for (int j = 0; j <= t; ++j) { p[j] = std::exp(p[j] - m); denom += p[j]; }
                for (int j = 0; j <= t; ++j)
                    for (int d = 0; d < hd; ++d)
                        a[((size_t)t * nq + g) * hd + d] += p[j] / denom * v[((size_t)j * nkv + kvh) * hd + d];
            }
        }
        const vec o = linear(a, wo.data(), T, nq * hd, H);
        for (size_t i = 0; i < h.size(); ++i) h[i] += o[i];
        // SwiGLU feed-forward: down(silu(gate x) * up x), silu(g) = g / (1 + exp(-g))
        // (prefill_engine.rs:3226-3366; full_attention_cuda.cuh:1995-2010)
        const vec x2 = rms_norm(h, ln2.data(), T, H, eps);
        vec gt = linear(x2, wg.data(), T, H, I);
        const vec up = linear(x2, wu.data(), T, H, I);
        for (size_t i = 0; i < gt.size(); ++i) gt[i] = gt[i] / (1.0 + std::exp(-gt[i])) * up[i];
        const vec dn = linear(gt, wd.data(), T, I, H);
        for (size_t i = 0; i < h.size(); ++i) h[i] += dn[i];
    }
    // final norm and head; a tied head reuses the embedding (prefill_engine.rs:515-640; llama31_engine.rs:184-192)
    const vec norm_w = read_vec(H);
    const vec n = rms_norm(h, norm_w.data(), T, H, eps);
    vec logits;
    if (tied) logits = linear(n, embed.data(), T, H, V);
    else { const vec head = read_vec((size_t)V * H); logits = linear(n, head.data(), T, H, V); }
    fclose(f);
    FILE* out = fopen(argv[2], "wb");
    if (!out || fwrite(logits.data(), sizeof(double), logits.size(), out) != logits.size()) { perror("write output"); return 1; }
    fclose(out);
    return 0;
}
