// Runs celsowm/celeg's own float32 CPU kernels on small fixed inputs and prints inputs and outputs as
// JSON. Built and run by make_golden.sh against the reference checkout; the result is committed as
// golden.json and compared with tests/plain_lfm2.py by tests/test_golden_reference.py.
#include "celeg/backend/cpu/kernels.hpp"
#include "celeg/backend/cpu/paged_kv.hpp"
#include "celeg/backend/cpu/sampler.hpp"
#include "celeg/model/definition.hpp"
#include "celeg/model/runtime_types.hpp"

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <vector>

static uint64_t g_state = 0x9E3779B97F4A7C15ull;
static float next_value() {                       // splitmix64 -> [-1, 1)
    uint64_t z = (g_state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return static_cast<float>((z >> 40) * (1.0 / 8388608.0) - 1.0);
}
static std::vector<float> values(size_t n, float scale = 1.0f) {
    std::vector<float> v(n);
    for (auto& x : v) x = next_value() * scale;
    return v;
}
static void print(const char* name, const std::vector<float>& v, bool last = false) {
    std::printf("  \"%s\": [", name);
    for (size_t i = 0; i < v.size(); ++i) std::printf("%s%.9g", i ? "," : "", v[i]);
    std::printf("]%s\n", last ? "" : ",");
}

int main() {
    std::printf("{\n");
    {   // RMSNorm, width 48, eps 1e-5
        auto x = values(48), w = values(48);
        std::vector<float> y(48);
        celeg::cpu_rmsnorm(x.data(), w.data(), y.data(), 48, 1e-5f);
        print("rmsnorm_x", x); print("rmsnorm_w", w); print("rmsnorm_y", y);
    }
    {   // SwiGLU on gate|up of 40 each
        auto gu = values(80, 3.0f);
        std::vector<float> y(40);
        celeg::cpu_swiglu(gu.data(), y.data(), 40);
        print("swiglu_gate_up", gu); print("swiglu_y", y);
    }
    {   // per-head RMSNorm + split-half RoPE: 3 heads of 16 at position 37, theta 10000, eps 1e-6
        auto x = values(48), w = values(16);
        auto y = x;
        celeg::RopePositionSpec rope;
        rope.theta = 10000.0;
        celeg::cpu_qk_norm_rope(y.data(), w.data(), 3, 16, 37, rope, 1e-6f);
        print("qk_x", x); print("qk_w", w); print("qk_y", y);
        std::printf("  \"qk_rotary_fraction\": %.9g,\n", static_cast<double>(rope.rotary_fraction));
    }
    {   // short convolution, 7 tokens one by one: hidden 10, kernel length 3, weights tap-major [tap][hidden]
        const int hidden = 10, taps = 3, tokens = 7;
        auto proj = values(static_cast<size_t>(tokens) * 3 * hidden);
        auto weight = values(static_cast<size_t>(taps) * hidden);
        std::vector<float> state(static_cast<size_t>(taps) * hidden, 0.0f), out(static_cast<size_t>(tokens) * hidden);
        for (int t = 0; t < tokens; ++t)
            celeg::cpu_conv_decode(proj.data() + static_cast<size_t>(t) * 3 * hidden, weight.data(), state.data(),
                                   out.data() + static_cast<size_t>(t) * hidden, hidden, taps, t);
        print("conv_proj", proj); print("conv_weight_tap_major", weight); print("conv_decode_out", out);
        // the same tokens as one chunk from position 0
        std::vector<float> state2(static_cast<size_t>(taps) * hidden, 0.0f), out2(out.size());
        celeg::CpuThreadPool pool(1);
        celeg::cpu_conv_prefill(proj.data(), weight.data(), state2.data(), out2.data(), tokens, hidden, taps, 0, pool);
        print("conv_prefill_out", out2);
    }
    {   // sampler: 12 draws at temperature 0.8, top_k 5, top_p 0.9, penalty 1.3, seed 7; then greedy
        const int vocab = 32;
        auto logits = values(vocab, 4.0f);
        std::vector<uint8_t> seen(vocab, 0);
        seen[3] = seen[11] = seen[20] = 1;
        celeg::GenerationConfig generation;
        generation.temperature = 0.8f;
        generation.top_k = 5;
        generation.top_p = 0.9f;
        generation.repetition_penalty = 1.3f;
        uint64_t rng = 7;
        std::vector<float> draws;
        for (int i = 0; i < 12; ++i)
            draws.push_back(static_cast<float>(celeg::CpuSampler::sample(logits, vocab, generation, seen, rng)));
        generation.temperature = 0.0f;
        draws.push_back(static_cast<float>(celeg::CpuSampler::sample(logits, vocab, generation, seen, rng)));
        print("sampler_logits", logits); print("sampler_draws", draws);
    }
    {   // causal grouped-query attention over a paged float32 cache: 4 query heads on 2 kv heads of 16, 21 keys
        // in pages of 8 (three pages, taken from the pool out of order), the query at the last position and the
        // same query at position 9, that is over a sequence of 10 keys ending inside the second page (celeg's
        // chunk attention calls the kernel once per row with that row's own sequence length:
        // src/backend/cpu/attention/paged_prefill.cpp:30). q, k and v are given as they are after norm and
        // rotation; the kernel applies 1/sqrt(head_dim) itself.
        const int q_heads = 4, kv_heads = 2, head_dim = 16, keys = 21, page_tokens = 8;
        auto q = values(static_cast<size_t>(q_heads) * head_dim, 2.0f);
        auto k = values(static_cast<size_t>(keys) * kv_heads * head_dim, 2.0f);
        auto v = values(static_cast<size_t>(keys) * kv_heads * head_dim);
        celeg::CpuKvPagePool pool(celeg::CpuKvCacheMode::Fp32, page_tokens,
                                  celeg::CpuOrdinaryKvPageLayout{static_cast<size_t>(kv_heads * head_dim),
                                                                 static_cast<size_t>(kv_heads * head_dim)});
        std::vector<celeg::CpuKvPageId> taken;
        for (int i = 0; i < 5; ++i) taken.push_back(pool.allocate());
        std::vector<celeg::CpuKvPageId> pages = {taken[3], taken[0], taken[4]};
        for (int t = 0; t < keys; ++t)
            pool.write(pages[static_cast<size_t>(t / page_tokens)], static_cast<size_t>(t % page_tokens),
                       k.data() + static_cast<size_t>(t) * kv_heads * head_dim,
                       v.data() + static_cast<size_t>(t) * kv_heads * head_dim);
        std::vector<float> last(static_cast<size_t>(q_heads) * head_dim), middle(last.size());
        celeg::cpu_gqa_decode_paged(q.data(), pool, pages, last.data(), keys, q_heads, kv_heads, head_dim);
        celeg::cpu_gqa_decode_paged(q.data(), pool, pages, middle.data(), 10, q_heads, kv_heads, head_dim);
        print("attention_q", q); print("attention_k", k); print("attention_v", v);
        print("attention_out_last", last); print("attention_out_at_9", middle, true);
    }
    std::printf("}\n");
    return 0;
}
