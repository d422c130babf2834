// A second plain implementation of the Llama-family decoder that Glassbox runs, in C++ and float32, written from
// the formulas of crates/glassbox-core/src/model.rs (each function cites file:line). It shares nothing with the
// glassbox_b200 package or its kernels and nothing with the NumPy implementation beside it: the two are compared
// with each other before either judges the engine. It also serves as the timed CPU baseline: like the reference it
// keeps everything in float32 (weights, activations, cache, accumulation; model.rs:228-243, kv.rs:17-19), computes
// each output as one dot product, and keeps a contiguous cache for one sequence.
//
// C ABI (loaded with ctypes by ref_forward.py): ref_new / ref_set / ref_forward / ref_free.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#define REF_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

struct Layer {
    const float *attn_norm, *wq, *wk, *wv, *wo, *mlp_norm, *w_gate, *w_up, *w_down;
};

struct Model {
    int d, inter, layers, nh, nkv, hd, vocab, max_pos;
    float eps, theta;
    const float *embed, *norm, *head;      // head == embed when tied (model.rs:190-192)
    std::vector<Layer> layer;
    std::vector<float> kcache, vcache;     // [layers][max_pos][nkv * hd], keys stored rotated (model.rs:273-275)
    std::vector<float> inv_freq;           // [hd / 2]
};

// A fork-join pool: par_for(n, f) runs f(i) for i in 0..n on REF_THREADS threads (default 4, the thread count of the
// reference's published numbers). Workers spin briefly for the next job, then sleep (the idea of
// crates/glassbox-core/src/pool.rs:1-7; the code is this file's own).
class Pool {
public:
    Pool() {
        const char* env = std::getenv("REF_THREADS");
        int n = env ? std::atoi(env) : 4;
        const int hw = (int)std::thread::hardware_concurrency();
        if (hw > 0 && n > hw) n = hw;
        if (n < 1) n = 1;
        for (int w = 1; w < n; ++w) workers_.emplace_back([this] { work(); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> g(mu_);
            stop_ = true;
            ++generation_;
        }
        cv_.notify_all();
        for (auto& t : workers_) t.join();
    }
    void run(int n, const std::function<void(int)>& f) {
        if (workers_.empty() || n < 2) {
            for (int i = 0; i < n; ++i) f(i);
            return;
        }
        {
            std::lock_guard<std::mutex> g(mu_);
            job_ = &f;
            total_ = n;
            next_.store(0);
            pending_.store((int)workers_.size());
            ++generation_;
        }
        cv_.notify_all();
        drain();
        while (pending_.load(std::memory_order_acquire) != 0) std::this_thread::yield();
    }

private:
    void drain() {
        for (;;) {
            const int i = next_.fetch_add(1);
            if (i >= total_) return;
            (*job_)(i);
        }
    }
    void work() {
        long seen = 0;
        for (;;) {
            int spins = 0;
            while (generation_.load(std::memory_order_acquire) == seen && ++spins < 20000) std::this_thread::yield();
            if (generation_.load(std::memory_order_acquire) == seen) {
                std::unique_lock<std::mutex> g(mu_);
                cv_.wait(g, [&] { return generation_.load() != seen; });
            }
            {
                std::lock_guard<std::mutex> g(mu_);   // the job's fields were written under this lock
                seen = generation_.load();
                if (stop_) return;
            }
            drain();
            pending_.fetch_sub(1, std::memory_order_release);
        }
    }
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable cv_;
    std::atomic<long> generation_{0};
    std::atomic<int> next_{0}, pending_{0};
    const std::function<void(int)>* job_ = nullptr;
    int total_ = 0;
    bool stop_ = false;
};

Pool& pool() {
    static Pool p;
    return p;
}

void par_for(int n, const std::function<void(int)>& f) { pool().run(n, f); }

// One output = one dot product, eight partial sums that are added at the end (the shape of the reference's AVX2
// kernel, crates/glassbox-core/src/kernels.rs:116-131), so that the compiler can vectorise it without being
// allowed to reorder anything itself.
float dot(const float* a, const float* b, int n) {
    float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int i = 0;
    for (; i + 8 <= n; i += 8)
        for (int j = 0; j < 8; ++j) s[j] += a[i + j] * b[i + j];
    float tail = 0.f;
    for (; i < n; ++i) tail += a[i] * b[i];
    return ((s[0] + s[1]) + (s[2] + s[3])) + ((s[4] + s[5]) + (s[6] + s[7])) + tail;
}

// out[t, r] = dot(x[t, :], w[r, :]) for a row-major [rows, cols] weight (kernels.rs:381, 586)
void matmul(float* out, const float* x, int n, const float* w, int rows, int cols) {
    const int strip = 16;                                     // rows per task
    par_for((rows + strip - 1) / strip, [&](int task) {
        const int r1 = std::min(rows, (task + 1) * strip);
        for (int r = task * strip; r < r1; ++r)
            for (int t = 0; t < n; ++t) out[(size_t)t * rows + r] = dot(x + (size_t)t * cols, w + (size_t)r * cols, cols);
    });
}

// model.rs:94-100: ms = sum(x^2) / d; s = 1 / sqrt(ms + eps); out = w * (x * s)
void rms_norm(float* out, const float* x, const float* w, int d, float eps) {
    float ss = 0.f;
    for (int i = 0; i < d; ++i) ss += x[i] * x[i];
    const float s = 1.0f / std::sqrt(ss / (float)d + eps);
    for (int i = 0; i < d; ++i) out[i] = w[i] * (x[i] * s);
}

// model.rs:102-115: half-split pairs (i, i + hd/2); the inverse frequency is formed in float64 and rounded to
// float32, the angle is a float32 product, sine and cosine are evaluated in float64 and rounded to float32.
void rope(float* x, int hd, int pos, const float* inv_freq) {
    const int half = hd / 2;
    for (int i = 0; i < half; ++i) {
        const float a = (float)pos * inv_freq[i];
        const float s = (float)std::sin((double)a), c = (float)std::cos((double)a);
        const float x0 = x[i], x1 = x[i + half];
        x[i] = x0 * c - x1 * s;
        x[i + half] = x1 * c + x0 * s;
    }
}

}  // namespace

// sizes: d, inter, layers, nh, nkv, hd, vocab, max_pos
REF_EXPORT void* ref_new(const int* sizes, float eps, float theta) {
    Model* m = new Model();
    m->d = sizes[0]; m->inter = sizes[1]; m->layers = sizes[2]; m->nh = sizes[3]; m->nkv = sizes[4];
    m->hd = sizes[5]; m->vocab = sizes[6]; m->max_pos = sizes[7];
    m->eps = eps; m->theta = theta;
    m->embed = m->norm = m->head = nullptr;
    m->layer.resize(m->layers);
    const size_t per = (size_t)m->max_pos * m->nkv * m->hd;
    m->kcache.assign(per * m->layers, 0.f);
    m->vcache.assign(per * m->layers, 0.f);
    m->inv_freq.resize(m->hd / 2);
    for (int i = 0; i < m->hd / 2; ++i)
        m->inv_freq[i] = (float)(1.0 / std::pow((double)theta, 2.0 * i / (double)m->hd));   // model.rs:107
    return m;
}

// which: 0 embed, 1 final norm, 2 head; per layer (layer >= 0): 0 attn_norm, 1 wq, 2 wk, 3 wv, 4 wo, 5 mlp_norm,
// 6 gate, 7 up, 8 down. The caller keeps the arrays alive.
REF_EXPORT void ref_set(void* h, int layer, int which, const float* data) {
    Model* m = static_cast<Model*>(h);
    if (layer < 0) {
        (which == 0 ? m->embed : which == 1 ? m->norm : m->head) = data;
        return;
    }
    Layer& l = m->layer[layer];
    const float** slot[] = {&l.attn_norm, &l.wq, &l.wk, &l.wv, &l.wo, &l.mlp_norm, &l.w_gate, &l.w_up, &l.w_down};
    *slot[which] = data;
}

REF_EXPORT void ref_free(void* h) { delete static_cast<Model*>(h); }

// model.rs:207-362 for one sequence: n tokens at positions pos0 .. pos0+n-1, everything before them in the cache
// that earlier calls left; logits [n_want, vocab] at the batch indices `want`. Returns 0, or 1 if the positions
// run past max_pos.
REF_EXPORT int ref_forward(void* h, const int* tokens, int n, int pos0, const int* want, int n_want, float* logits) {
    Model* m = static_cast<Model*>(h);
    const int d = m->d, nh = m->nh, nkv = m->nkv, hd = m->hd, inter = m->inter;
    const int qd = nh * hd, kvd = nkv * hd, group = nh / nkv;
    if (pos0 < 0 || pos0 + n > m->max_pos) return 1;
    std::vector<float> x((size_t)n * d), hbuf((size_t)n * d), q((size_t)n * qd), k((size_t)n * kvd), v((size_t)n * kvd),
        att((size_t)n * qd), o((size_t)n * d), gate((size_t)n * inter), up((size_t)n * inter);
    for (int i = 0; i < n; ++i)                                                        // model.rs:228-231
        std::memcpy(&x[(size_t)i * d], m->embed + (size_t)tokens[i] * d, sizeof(float) * d);
    const float scale = 1.0f / std::sqrt((float)hd);                                   // model.rs:244
    for (int li = 0; li < m->layers; ++li) {
        const Layer& l = m->layer[li];
        float* kc = &m->kcache[(size_t)li * m->max_pos * kvd];
        float* vc = &m->vcache[(size_t)li * m->max_pos * kvd];
        for (int i = 0; i < n; ++i) rms_norm(&hbuf[(size_t)i * d], &x[(size_t)i * d], l.attn_norm, d, m->eps);   // 252-259
        matmul(q.data(), hbuf.data(), n, l.wq, qd, d);                                 // model.rs:260-265
        matmul(k.data(), hbuf.data(), n, l.wk, kvd, d);
        matmul(v.data(), hbuf.data(), n, l.wv, kvd, d);
        for (int i = 0; i < n; ++i) {                                                  // model.rs:266-276
            for (int hh = 0; hh < nh; ++hh) rope(&q[(size_t)i * qd + hh * hd], hd, pos0 + i, m->inv_freq.data());
            for (int hh = 0; hh < nkv; ++hh) rope(&k[(size_t)i * kvd + hh * hd], hd, pos0 + i, m->inv_freq.data());
            std::memcpy(kc + (size_t)(pos0 + i) * kvd, &k[(size_t)i * kvd], sizeof(float) * kvd);
            std::memcpy(vc + (size_t)(pos0 + i) * kvd, &v[(size_t)i * kvd], sizeof(float) * kvd);
        }
        par_for(n * nh, [&](int task) {                                                // model.rs:278-317
                const int i = task / nh, hh = task % nh;
                const int kvh = hh / group, ctx = pos0 + i + 1;
                const float* qv = &q[(size_t)i * qd + hh * hd];
                std::vector<float> score(ctx);
                float mx = -INFINITY;
                for (int p = 0; p < ctx; ++p) {
                    score[p] = dot(qv, kc + (size_t)p * kvd + kvh * hd, hd) * scale;
                    mx = std::fmax(mx, score[p]);
                }
                float z = 0.f;
                for (int p = 0; p < ctx; ++p) {
                    score[p] = std::exp(score[p] - mx);
                    z += score[p];
                }
                float* out = &att[(size_t)i * qd + hh * hd];
                for (int c = 0; c < hd; ++c) out[c] = 0.f;
                for (int p = 0; p < ctx; ++p) {
                    const float prob = score[p] / z;                                   // normalised before the sum
                    const float* vv = vc + (size_t)p * kvd + kvh * hd;
                    for (int c = 0; c < hd; ++c) out[c] += prob * vv[c];
                }
        });
        matmul(o.data(), att.data(), n, l.wo, d, qd);                                  // model.rs:322-325
        for (size_t i = 0; i < (size_t)n * d; ++i) x[i] += o[i];
        for (int i = 0; i < n; ++i) rms_norm(&hbuf[(size_t)i * d], &x[(size_t)i * d], l.mlp_norm, d, m->eps);    // 327-334
        matmul(gate.data(), hbuf.data(), n, l.w_gate, inter, d);                       // model.rs:335
        matmul(up.data(), hbuf.data(), n, l.w_up, inter, d);
        for (size_t i = 0; i < (size_t)n * inter; ++i) gate[i] = gate[i] / (1.0f + std::exp(-gate[i])) * up[i];   // 336-340
        matmul(o.data(), gate.data(), n, l.w_down, d, inter);                          // model.rs:341-344
        for (size_t i = 0; i < (size_t)n * d; ++i) x[i] += o[i];
    }
    std::vector<float> hs((size_t)std::max(n_want, 1) * d);
    for (int j = 0; j < n_want; ++j) rms_norm(&hs[(size_t)j * d], &x[(size_t)want[j] * d], m->norm, d, m->eps);  // 350-358
    matmul(logits, hs.data(), n_want, m->head, m->vocab, d);                           // model.rs:359-361
    return 0;
}
