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
// Every reduction has a fixed shape (a warp owns a contiguous run of the vocabulary, then a serial scan over the
// warps' sums, then a scan over the lanes), so a row's result never depends on the other rows.
#include "common.cuh"

#include <float.h>

constexpr int SAMPLE_THREADS = 512;

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* __restrict__ logits, long long stride,
                                                                const float* __restrict__ temperature,
                                                                const float* __restrict__ uniform,
                                                                const int* __restrict__ want_slots,
                                                                unsigned* __restrict__ state, int num_slots,
                                                                int* __restrict__ last_token,
                                                                int* __restrict__ out, int vocab) {
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* l = logits + (size_t)row * stride;
    __shared__ float s_val[SAMPLE_THREADS];
    __shared__ int s_idx[SAMPLE_THREADS];
    __shared__ float s_pref[SAMPLE_THREADS + 1];

    // Maximum and its first index: coalesced strided reads, ties go to the lower index.
    float best = -FLT_MAX;
    int best_i = vocab;
    if (vocab % 4 == 0 && ((uintptr_t)l & 15) == 0) {
        // twelve 16-byte loads in flight per thread (instructions issue in order: a value used as soon as it is asked
        // for costs the whole trip to memory every time round); a thread's indices still ascend
        const float4* l4 = reinterpret_cast<const float4*>(l);
        const int n4 = vocab / 4;
        constexpr int FLY = 12;   // 16-byte loads in flight per thread
        for (int i0 = tid; i0 < n4; i0 += FLY * SAMPLE_THREADS) {
            float4 v[FLY];
#pragma unroll
            for (int u = 0; u < FLY; ++u) {
                const int i = i0 + u * SAMPLE_THREADS;
                v[u] = i < n4 ? l4[i] : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
            }
#pragma unroll
            for (int u = 0; u < FLY; ++u) {
                const int i = (i0 + u * SAMPLE_THREADS) * 4;
                if (i >= vocab) continue;
                if (best_i == vocab || v[u].x > best) { best = v[u].x; best_i = i; }
                if (v[u].y > best) { best = v[u].y; best_i = i + 1; }
                if (v[u].z > best) { best = v[u].z; best_i = i + 2; }
                if (v[u].w > best) { best = v[u].w; best_i = i + 3; }
            }
        }
    } else {
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
            float v = l[i];
            if (best_i == vocab || v > best) { best = v; best_i = i; }   // i ascends, so ties keep the lower index
        }
    }
    // the maximum with its first index: inside each warp with shuffles, then over the sixteen warps (ties: lower index)
    auto better = [&](float ov, int oi, float cv, int ci) { return oi < vocab && (ci == vocab || ov > cv || (ov == cv && oi < ci)); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_down_sync(0xffffffffu, best, o);
        const int oi = __shfl_down_sync(0xffffffffu, best_i, o);
        if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    if ((tid & 31) == 0) {
        s_val[tid >> 5] = best;
        s_idx[tid >> 5] = best_i;
    }
    __syncthreads();
    if (tid < 32) {
        float cv = tid < SAMPLE_THREADS / 32 ? s_val[tid] : -FLT_MAX;
        int ci = tid < SAMPLE_THREADS / 32 ? s_idx[tid] : vocab;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_down_sync(0xffffffffu, cv, o);
            const int oi = __shfl_down_sync(0xffffffffu, ci, o);
            if (better(ov, oi, cv, ci)) { cv = ov; ci = oi; }
        }
        if (tid == 0) {
            s_val[0] = cv;
            s_idx[0] = ci;
        }
    }
    __syncthreads();
    const float vmax = s_val[0];
    const int imax = s_idx[0];
    __shared__ float s_draw[2];   // temperature, uniform
    __shared__ int s_slot;
    if (tid == 0) {
        float temp0 = temperature ? temperature[row] : 0.f, r = uniform ? uniform[row] : 0.f;
        const int slot = want_slots ? want_slots[row] : -1;
        s_slot = (slot >= 0 && slot < num_slots && last_token != nullptr) ? slot : -1;
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
        if (tid == 0) {
            out[row] = imax;
            if (s_slot >= 0) last_token[s_slot] = imax;
        }
        return;
    }
    // Temperature: every warp owns a contiguous run of the vocabulary and reads it coalesced. First the runs' sums
    // (and a serial scan over the sixteen of them), then the one warp whose run holds the target walks it, 32 tokens
    // at a time, with a scan over its lanes: the walk is in token order, and each pass reads a row once.
    const float inv_temp = 1.0f / temp;   // exp((l - max) / temperature): the maximum subtracted before the division
    const int lane = tid & 31, warp = tid >> 5;
    constexpr int WARPS = SAMPLE_THREADS / 32;
    const int run = ((vocab + WARPS - 1) / WARPS + 31) / 32 * 32;
    const int wlo = min(warp * run, vocab), whi = min(wlo + run, vocab);
    float part = 0.f;
    for (int i = wlo + lane; i < whi; i += 32) part += __expf((l[i] - vmax) * inv_temp);
    part = gb_warp_sum(part);
    if (lane == 0) s_val[warp] = part;
    __syncthreads();
    if (tid == 0) {
        float acc = 0.f;
        for (int w = 0; w < WARPS; ++w) {
            s_pref[w] = acc;
            acc += s_val[w];
        }
        s_pref[WARPS] = acc;
        out[row] = max(vocab - 1, 0);  // fallback: the last token, as sampler.rs:163
        if (s_slot >= 0) last_token[s_slot] = max(vocab - 1, 0);
    }
    __syncthreads();
    const float target = s_draw[1] * s_pref[WARPS];
    // Exactly one warp's half-open interval [pref, pref + sum) holds the target (if any does). Inside its run every lane
    // takes a contiguous piece: the lanes' sums, one scan over them, and the one lane whose piece holds the target walks it.
    if (wlo < whi && target >= s_pref[warp] && target < s_pref[warp + 1]) {
        const int piece = (whi - wlo + 31) / 32;
        const int plo = min(wlo + lane * piece, whi), phi = min(plo + piece, whi);
        float mine = 0.f;
        for (int i = plo; i < phi; ++i) mine += __expf((l[i] - vmax) * inv_temp);
        float upto = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {   // inclusive scan over the lanes, in token order
            const float up = __shfl_up_sync(0xffffffffu, upto, o);
            if (lane >= o) upto += up;
        }
        const float before = s_pref[warp] + upto - mine;
        const unsigned hit = __ballot_sync(0xffffffffu, plo < phi && target < before + mine);
        // the first lane whose piece reaches past the target; rounding may leave none: then the run's last token
        const int owner = hit ? __ffs(hit) - 1 : -1;
        int pick = whi - 1;
        if (lane == owner) {
            float acc = before;
            pick = phi - 1;
            for (int i = plo; i < phi; ++i) {
                acc += __expf((l[i] - vmax) * inv_temp);
                if (target < acc) { pick = i; break; }
            }
        }
        if (lane == (owner >= 0 ? owner : 0)) {
            out[row] = pick;
            if (s_slot >= 0) last_token[s_slot] = pick;
        }
    }
}

// tokens[i] = last_token[token_slots[i]] where token_slots[i] >= 0: a row whose token is the one the sampling kernel chose
// for its request in the step before, taken on the device (the host launched this step before it had read that token).
__global__ void resolve_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ token_slots,
                                      const int* __restrict__ last_token, int n, int num_slots) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int slot = token_slots[i];
    if (slot >= 0 && slot < num_slots) tokens[i] = last_token[slot];
}

GB_EXPORT int gb_resolve_tokens(int* tokens, const int* token_slots, const int* last_token, int n, int num_slots,
                                cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && tokens && token_slots && last_token && num_slots > 0, "gb_resolve_tokens: bad arguments");
    if (n == 0) return 0;
    resolve_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, token_slots, last_token, n, num_slots);
    return gb_check_launch("gb_resolve_tokens");
}

// temperature / uniform: per-row arrays (or null: greedy). want_slots / state: per-row state slot (-1: use the arrays)
// and the [num_slots, 4] sampling states (or null). last_token (or null): [num_slots], receives the chosen token of
// every row that names a slot, so that the next step can take it from there without the host in between.
GB_EXPORT int gb_sample(const float* logits, long long stride, const float* temperature, const float* uniform,
                        const int* want_slots, void* state, int num_slots, int* last_token, int* out, int rows, int vocab,
                        cudaStream_t stream) {
    GB_REQUIRE(rows >= 0 && vocab > 0 && stride >= vocab, "gb_sample: bad sizes rows=%d vocab=%d", rows, vocab);
    GB_REQUIRE(temperature == nullptr || uniform != nullptr, "gb_sample: temperature sampling needs uniform draws");
    GB_REQUIRE(want_slots == nullptr || (state != nullptr && num_slots > 0), "gb_sample: state slots need the sampling states");
    if (rows == 0) return 0;
    sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, stride, temperature, uniform, want_slots, (unsigned*)state,
                                                        num_slots, last_token, out, vocab);
    return gb_check_launch("gb_sample");
}
