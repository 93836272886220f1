// Calls the reference's own CPU operators (src/qwen_ops.cpp, src/sampler.cpp, compiled unmodified) on
// fixed pseudo-random inputs and prints inputs and outputs as JSON.  Built and run by make_golden.py;
// `hip/hip_fp16.h` is replaced by the small shim that script writes (a float-backed __half).
#include "qwen_ops.h"
#include "sampler.h"

#include <cstdio>
#include <cstdint>
#include <vector>

static uint64_t state = 88172645463325252ull;
static float rnd() {  // xorshift, uniform in [-1, 1)
    state ^= state << 13; state ^= state >> 7; state ^= state << 17;
    return (float)((state >> 11) * (1.0 / 9007199254740992.0)) * 2.0f - 1.0f;
}
static void dump(const char* name, const std::vector<float>& v, bool last = false) {
    printf("\"%s\": [", name);
    for (size_t i = 0; i < v.size(); ++i) printf("%s%.9g", i ? ", " : "", v[i]);
    printf("]%s\n", last ? "" : ",");
}

int main() {
    printf("{\n");
    {   // RMSNorm, n = 96, eps 1e-5
        const int n = 96;
        std::vector<float> x(n), w(n), y(n);
        for (auto& v : x) v = rnd() * 3.0f;
        for (auto& v : w) v = 1.0f + 0.2f * rnd();
        qwen_rmsnorm(x.data(), w.data(), y.data(), n, 1e-5f);
        dump("rms_x", x); dump("rms_w", w); dump("rms_y", y);
    }
    {   // rotate-half RoPE, head_dim 32, n_rot 32 and 16, positions 0, 7, 1234
        const int d = 32;
        std::vector<float> v0(d);
        for (auto& v : v0) v = rnd();
        dump("rope_in", v0);
        const int pos[3] = {0, 7, 1234};
        for (int i = 0; i < 3; ++i) {
            std::vector<float> a = v0, b = v0;
            qwen_rope_neox(a.data(), 32, pos[i], 1e6f);
            qwen_rope_neox(b.data(), 16, pos[i], 10000.0f);
            char name[64];
            snprintf(name, sizeof name, "rope_full_theta1e6_pos%d", pos[i]); dump(name, a);
            snprintf(name, sizeof name, "rope_half_theta1e4_pos%d", pos[i]); dump(name, b);
        }
    }
    {   // single-query GQA attention: 8 heads, 2 kv heads, head_dim 32, 37 cached positions
        const int H = 8, HKV = 2, D = 32, N = 37, stride = HKV * D;
        std::vector<float> q(H * D), kf(N * stride), vf(N * stride), out(H * D);
        for (auto& v : q) v = rnd() * 2.0f;
        for (auto& v : kf) v = rnd();
        for (auto& v : vf) v = rnd();
        std::vector<__half> K(kf.size()), V(vf.size());
        for (size_t i = 0; i < kf.size(); ++i) { K[i] = __float2half(kf[i]); V[i] = __float2half(vf[i]); }
        qwen_attention(q.data(), K.data(), V.data(), stride, N, H, HKV, D, 0.17677669529663687f, out.data());
        dump("attn_q", q); dump("attn_k", kf); dump("attn_v", vf); dump("attn_out", out);
    }
    {   // SiLU
        std::vector<float> x(16), y(16);
        for (auto& v : x) v = rnd() * 6.0f;
        for (int i = 0; i < 16; ++i) y[i] = qwen_silu(x[i]);
        dump("silu_x", x); dump("silu_y", y);
    }
    {   // sampler: logits over 64 tokens; greedy with a tie, and seeded draws for four chains
        const int n = 64;
        std::vector<float> l(n);
        for (auto& v : l) v = rnd() * 4.0f;
        l[40] = l[11] = 9.0f;                       // a tie: the lower id must win
        dump("samp_logits", l);
        sampler_params p = sampler_default_params();
        p.temperature = 0.0f;
        sampler_t* s = sampler_create(&p);
        printf("\"samp_greedy\": %d,\n", sampler_sample(s, l.data(), n));
        sampler_free(s);
        struct { const char* name; float t; int k; float tp, mp, rp, pp; uint64_t seed; } cases[] = {
            {"samp_default_seed3", 0.8f, 40, 0.95f, 0.05f, 1.0f, 0.0f, 3},
            {"samp_temp_only_seed1", 0.7f, 0, 1.0f, 0.0f, 1.0f, 0.0f, 1},
            {"samp_topp_only_seed5", 1.3f, 0, 0.6f, 0.0f, 1.0f, 0.0f, 5},
            {"samp_penalty_seed9", 1.0f, 10, 1.0f, 0.0f, 1.3f, 0.5f, 9},
        };
        for (auto& c : cases) {
            p = sampler_default_params();
            p.temperature = c.t; p.top_k = c.k; p.top_p = c.tp; p.min_p = c.mp; p.repeat_penalty = c.rp;
            p.presence_penalty = c.pp; p.seed = c.seed;
            s = sampler_create(&p);
            printf("\"%s\": [", c.name);
            for (int i = 0; i < 40; ++i) {
                const int t = sampler_sample(s, l.data(), n);
                sampler_accept(s, t);
                printf("%s%d", i ? ", " : "", t);
            }
            printf("],\n");
            sampler_free(s);
        }
    }
    printf("\"end\": 0\n}\n");
    return 0;
}
