// Next-token choice on the device: greedy argmax and temperature sampling, one block per row.
//
// Greedy: the first maximum wins (crates/glassbox-core/src/sampler.rs:49-57).
// Temperature: logits are divided by the temperature, soft-maxed with the maximum subtracted
// (sampler.rs:113-125) and the token is drawn by walking the cumulative sum until it passes
// r * sum, with r in [0, 1) supplied per row by the host's xorshift64* generator
// (sampler.rs:150-164). The walk goes in token-id order; Glassbox walks candidates sorted by
// probability, which gives the same distribution but another token for the same r.
// A row's temperature and random number come either from the arrays the caller passes, or from the sampling state of
// the row's request: four 32-bit words per state slot, {generator state low, high, temperature bits, unused}, kept on
// the device beside the request's other per-request state. The kernel then advances the request's xorshift64*
// generator itself (sampler.rs:31-47: x ^= x >> 12; x ^= x << 25; x ^= x >> 27; r = (x * 0x2545f4914f6cdd1d) >> 40,
// r / 2^24), once per sampled token, so that nothing has to be drawn on the host for a step.
// Every reduction has a fixed shape (thread t owns a contiguous run of the vocabulary, then a
// serial scan over the threads' sums), so a row's result never depends on the other rows.
#include "common.cuh"

#include <float.h>

constexpr int SAMPLE_THREADS = 512;

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* __restrict__ logits, long long stride,
                                                                const float* __restrict__ temperature,
                                                                const float* __restrict__ uniform,
                                                                const int* __restrict__ want_slots,
                                                                unsigned* __restrict__ state, int num_slots,
                                                                int* __restrict__ out, int vocab) {
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* l = logits + (size_t)row * stride;
    const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int lo = min(tid * chunk, vocab), hi = min(lo + chunk, vocab);
    __shared__ float s_val[SAMPLE_THREADS];
    __shared__ int s_idx[SAMPLE_THREADS];
    __shared__ float s_pref[SAMPLE_THREADS + 1];

    // Maximum and its first index: coalesced strided reads, ties go to the lower index.
    float best = -FLT_MAX;
    int best_i = vocab;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        float v = l[i];
        if (best_i == vocab || v > best) { best = v; best_i = i; }   // i ascends, so ties keep the lower index
    }
    s_val[tid] = best;
    s_idx[tid] = best_i;
    __syncthreads();
    for (int s = SAMPLE_THREADS / 2; s > 0; s >>= 1) {
        if (tid < s) {
            float ov = s_val[tid + s];
            int oi = s_idx[tid + s];
            const int ci = s_idx[tid];
            if (oi < vocab && (ci == vocab || ov > s_val[tid] || (ov == s_val[tid] && oi < ci))) {  // ties: lower index
                s_val[tid] = ov;
                s_idx[tid] = oi;
            }
        }
        __syncthreads();
    }
    const float vmax = s_val[0];
    const int imax = s_idx[0];
    __shared__ float s_draw[2];   // temperature, uniform
    if (tid == 0) {
        float temp0 = temperature ? temperature[row] : 0.f, r = uniform ? uniform[row] : 0.f;
        const int slot = want_slots ? want_slots[row] : -1;
        if (slot >= 0 && slot < num_slots) {   // the request's own state: its temperature, and the next draw of its generator
            unsigned* st = state + 4 * (size_t)slot;
            temp0 = __uint_as_float(st[2]);
            if (temp0 > 0.f) {
                unsigned long long x = ((unsigned long long)st[1] << 32) | st[0];
                x ^= x >> 12;
                x ^= x << 25;
                x ^= x >> 27;
                st[0] = (unsigned)x;
                st[1] = (unsigned)(x >> 32);
                r = (float)((x * 0x2545F4914F6CDD1Dull) >> 40) / 16777216.0f;
            }
        }
        s_draw[0] = temp0;
        s_draw[1] = r;
    }
    __syncthreads();
    const float temp = s_draw[0];
    if (!(temp > 0.f)) {
        if (tid == 0) out[row] = imax;
        return;
    }
    const float mscaled = vmax / temp;
    float part = 0.f;
    for (int i = lo; i < hi; ++i) part += expf(l[i] / temp - mscaled);
    s_val[tid] = part;
    __syncthreads();
    if (tid == 0) {
        float run = 0.f;
        for (int t = 0; t < SAMPLE_THREADS; ++t) {
            s_pref[t] = run;
            run += s_val[t];
        }
        s_pref[SAMPLE_THREADS] = run;
        out[row] = max(vocab - 1, 0);  // fallback: the last token, as sampler.rs:163
    }
    __syncthreads();
    const float target = s_draw[1] * s_pref[SAMPLE_THREADS];
    // Exactly one thread's half-open interval [pref, pref + part) holds the target (if any does).
    if (lo < hi && target >= s_pref[tid] && target < s_pref[tid + 1]) {
        float run = s_pref[tid];
        int pick = hi - 1;
        for (int i = lo; i < hi; ++i) {
            run += expf(l[i] / temp - mscaled);
            if (target < run) { pick = i; break; }
        }
        out[row] = pick;
    }
}

// temperature / uniform: per-row arrays (or null: greedy). want_slots / state: per-row state slot (-1: use the arrays)
// and the [num_slots, 4] sampling states (or null).
GB_EXPORT int gb_sample(const float* logits, long long stride, const float* temperature, const float* uniform,
                        const int* want_slots, void* state, int num_slots, int* out, int rows, int vocab,
                        cudaStream_t stream) {
    GB_REQUIRE(rows >= 0 && vocab > 0 && stride >= vocab, "gb_sample: bad sizes rows=%d vocab=%d", rows, vocab);
    GB_REQUIRE(temperature == nullptr || uniform != nullptr, "gb_sample: temperature sampling needs uniform draws");
    GB_REQUIRE(want_slots == nullptr || (state != nullptr && num_slots > 0), "gb_sample: state slots need the sampling states");
    if (rows == 0) return 0;
    sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, stride, temperature, uniform, want_slots, (unsigned*)state,
                                                        num_slots, out, vocab);
    return gb_check_launch("gb_sample");
}
