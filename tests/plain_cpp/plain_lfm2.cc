// A second plain LFM2, in C++, for tests only: one token at a time with a growing
// list of keys and values and a ring of the last convolution inputs, as the
// reference's CPU path walks a sequence (crates/cellm-model/src/lfm.rs:263-763),
// in double precision for the tests and in 32-bit for the timed CPU baseline. It shares no code with the package nor with the
// Python plain implementation beside it (which works on whole sequences), so a
// slip in reading the reference would have to be made twice, in two forms, to
// go unseen. Each function cites the lines it restates.
//
// Built by tests/test_plain.py and by tests/plain_cpp/time_cpu_baseline.py with the host compiler; called through ctypes.
#include <cmath>
#include <cstddef>
#include <vector>

namespace {

struct Config {
    int vocab, hidden, layers, heads, kv_heads, head_dim, ff, taps;
    double eps, theta;
};

// Tensors of one layer, in the order the caller passes them.
enum Slot { OPERATOR_NORM, FFN_NORM, W1, W2, W3, IN_PROJ, CONV_W, CONV_B, OUT_PROJ, WQ, WK, WV, WO, Q_NORM, K_NORM, SLOTS };

// crates/cellm-kernels/src/cpu_kernels.rs:17-34: ms = sum x^2 / n; out = x / sqrt(ms + eps) * w (weight as it is).
template <typename R>
void rms_norm(const R* x, const R* w, int n, double eps, R* out) {
    R ss = 0;
    for (int i = 0; i < n; ++i) ss += x[i] * x[i];
    const R inv = (R)1 / std::sqrt(ss / n + (R)eps);
    for (int i = 0; i < n; ++i) out[i] = x[i] * inv * w[i];
}

// out[r] = sum_c W[r][c] x[c], W row-major [rows, cols], no bias (crates/cellm-model/src/lfm.rs:952-1000).
template <typename R>
void linear(const R* W, const R* x, int rows, int cols, R* out) {
    for (int r = 0; r < rows; ++r) {
        R acc = 0;
        const R* wr = W + (size_t)r * cols;
        for (int c = 0; c < cols; ++c) acc += wr[c] * x[c];
        out[r] = acc;
    }
}

// crates/cellm-kernels/src/cpu_kernels.rs:264-277 with rotary_dim = head_dim: pairs (i, i + hd/2).
template <typename R>
void rope(R* h, int hd, int pos, double theta) {
    const int half = hd / 2;
    for (int i = 0; i < half; ++i) {
        const R inv_freq = (R)std::pow((R)theta, (R)(-(2.0 * i) / hd));
        const R a = pos * inv_freq, c = std::cos(a), s = std::sin(a);
        const R x0 = h[i], x1 = h[half + i];
        h[i] = x0 * c - x1 * s;
        h[half + i] = x1 * c + x0 * s;
    }
}


// Logits [T, vocab] of one sequence. `w`: embed, final norm, head (null: the embedding is the
// head; an untied head is an addition to the reference, which always ties: lfm.rs:689-757), then
// SLOTS pointers per layer (null where the layer kind has no such tensor). `is_attention[l]`
// chooses the mixer. Returns 0, or -1 for a token id outside the vocabulary (lfm.rs:817-890).
template <typename R>
int forward(const Config* cfg, const R* const* w, const int* is_attention, const int* ids, int T, R* logits) {
    const Config& c = *cfg;
    const int H = c.hidden, hd = c.head_dim, A = c.heads * hd, KV = c.kv_heads * hd, ks = c.taps;
    const R* embed = w[0];
    const R* final_norm = w[1];
    const R* head = w[2] ? w[2] : w[0];
    // per layer: the keys and values of all tokens so far, or the last `taps` columns of B*x
    std::vector<std::vector<R>> keys(c.layers), values(c.layers), conv_state(c.layers);
    for (int l = 0; l < c.layers; ++l)
        if (!is_attention[l]) conv_state[l].assign((size_t)ks * H, (R)0);
    std::vector<R> x(H), xn(H), mix(H), bcx(3 * H), y(H), q(A), k(KV), v(KV), att(A), g(c.ff), u(c.ff), d(H), s;
    for (int t = 0; t < T; ++t) {
        if (ids[t] < 0 || ids[t] >= c.vocab) return -1;
        for (int i = 0; i < H; ++i) x[i] = embed[(size_t)ids[t] * H + i];
        for (int l = 0; l < c.layers; ++l) {
            const R* const* lw = w + 3 + (size_t)l * SLOTS;
            rms_norm(x.data(), lw[OPERATOR_NORM], H, c.eps, xn.data());                  // lfm.rs:333-347
            if (!is_attention[l]) {
                // lfm.rs:350-417: in_proj -> B | C | x; bx = B*x; the state shifts by one column and
                // takes bx; tap ks-1 meets the current token, tap 0 the oldest (:388-398); y = C*conv.
                linear(lw[IN_PROJ], xn.data(), 3 * H, H, bcx.data());
                std::vector<R>& st = conv_state[l];
                for (int ch = 0; ch < H; ++ch) {
                    for (int j = 0; j + 1 < ks; ++j) st[(size_t)ch * ks + j] = st[(size_t)ch * ks + j + 1];
                    st[(size_t)ch * ks + ks - 1] = bcx[ch] * bcx[2 * H + ch];
                    R conv = lw[CONV_B] ? lw[CONV_B][ch] : (R)0;                      // the bias is an addition
                    for (int j = 0; j < ks; ++j) conv += lw[CONV_W][(size_t)ch * ks + j] * st[(size_t)ch * ks + j];
                    y[ch] = bcx[H + ch] * conv;
                }
                linear(lw[OUT_PROJ], y.data(), H, H, mix.data());
            } else {
                // lfm.rs:418-601: q, k, v; per-head RMSNorm of q and k (:486-543); rope (:553-559); the
                // new key and value join the cache; head h reads key/value head h / (heads / kv_heads)
                // with scores q.k / sqrt(hd) over all cached tokens (kvcache.rs:710-790), softmax with
                // the maximum taken off (:1206-1227).
                linear(lw[WQ], xn.data(), A, H, q.data());
                linear(lw[WK], xn.data(), KV, H, k.data());
                linear(lw[WV], xn.data(), KV, H, v.data());
                std::vector<R> tmp(hd);
                for (int h = 0; h < c.heads; ++h) {
                    rms_norm(&q[(size_t)h * hd], lw[Q_NORM], hd, c.eps, tmp.data());
                    for (int i = 0; i < hd; ++i) q[(size_t)h * hd + i] = tmp[i];
                    rope(&q[(size_t)h * hd], hd, t, c.theta);
                }
                for (int h = 0; h < c.kv_heads; ++h) {
                    rms_norm(&k[(size_t)h * hd], lw[K_NORM], hd, c.eps, tmp.data());
                    for (int i = 0; i < hd; ++i) k[(size_t)h * hd + i] = tmp[i];
                    rope(&k[(size_t)h * hd], hd, t, c.theta);
                }
                keys[l].insert(keys[l].end(), k.begin(), k.end());
                values[l].insert(values[l].end(), v.begin(), v.end());
                const int group = c.heads / c.kv_heads;
                const R scale = (R)1 / std::sqrt((R)hd);
                s.resize(t + 1);
                for (int h = 0; h < c.heads; ++h) {
                    const int kvh = h / group;
                    R mx = -INFINITY;
                    for (int j = 0; j <= t; ++j) {
                        R dot = 0;
                        for (int i = 0; i < hd; ++i) dot += q[(size_t)h * hd + i] * keys[l][(size_t)j * KV + (size_t)kvh * hd + i];
                        s[j] = dot * scale;
                        mx = s[j] > mx ? s[j] : mx;
                    }
                    R sum = 0;
                    for (int j = 0; j <= t; ++j) { s[j] = std::exp(s[j] - mx); sum += s[j]; }
                    for (int i = 0; i < hd; ++i) {
                        R acc = 0;
                        for (int j = 0; j <= t; ++j) acc += s[j] * values[l][(size_t)j * KV + (size_t)kvh * hd + i];
                        att[(size_t)h * hd + i] = acc / sum;
                    }
                }
                linear(lw[WO], att.data(), H, A, mix.data());
            }
            for (int i = 0; i < H; ++i) x[i] += mix[i];                                  // lfm.rs:610-612
            rms_norm(x.data(), lw[FFN_NORM], H, c.eps, xn.data());                       // lfm.rs:615-629
            linear(lw[W1], xn.data(), c.ff, H, g.data());                               // lfm.rs:631-662
            linear(lw[W3], xn.data(), c.ff, H, u.data());
            for (int i = 0; i < c.ff; ++i) g[i] = g[i] * ((R)1 / ((R)1 + std::exp(-g[i]))) * u[i];
            linear(lw[W2], g.data(), H, c.ff, d.data());
            for (int i = 0; i < H; ++i) x[i] += d[i];                                    // lfm.rs:665-667
        }
        rms_norm(x.data(), final_norm, H, c.eps, xn.data());                             // lfm.rs:670-687
        linear(head, xn.data(), c.vocab, H, logits + (size_t)t * c.vocab);               // lfm.rs:689-757
    }
    return 0;
}
}  // namespace

// In double precision: the tests' second restatement.
extern "C" int plain_lfm2_forward(const Config* cfg, const double* const* w, const int* is_attention, const int* ids, int T,
                                  double* logits) {
    return forward<double>(cfg, w, is_attention, ids, T, logits);
}

// In 32-bit, as the reference's CPU path computes (crates/cellm-model/src/lfm.rs works on f32 throughout): the
// timed CPU baseline (tests/plain_cpp/time_cpu_baseline.py).
extern "C" int plain_lfm2_forward_f32(const Config* cfg, const float* const* w, const int* is_attention, const int* ids, int T,
                                      float* logits) {
    return forward<float>(cfg, w, is_attention, ids, T, logits);
}
