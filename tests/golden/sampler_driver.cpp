// Draws tokens from the reference's own sampler (core/src/sampling.cpp, compiled beside this
// file, not copied) on logits made by a small generator that the Python test repeats, and prints
// one JSON object: for every case its parameters and how often each token was drawn.  The
// reference seeds its generator from std::random_device, so single draws cannot be repeated;
// what is kept is the histogram of many draws (exact for greedy cases, which draw nothing).
#include <cstdint>
#include <cstdio>
#include <vector>

#include "core/sampling.h"

static uint32_t lcg_state;
static float next_logit() {            // 32-bit LCG (Numerical Recipes constants), top 16 bits
    lcg_state = lcg_state * 1664525u + 1013904223u;
    return ((lcg_state >> 16) / 65536.0f) * 8.0f - 4.0f;
}

struct Case { float temperature; int top_k; float top_p; float penalty; int n_prev; };

int main() {
    const int vocab = 50, draws = 40000;
    const Case cases[] = {
        {0.0f, 0, 1.0f, 1.0f, 0},  {0.0f, 0, 1.0f, 1.8f, 6},  {0.0f, 5, 0.5f, 3.0f, 12},
        {1.0f, 0, 1.0f, 1.0f, 0},  {0.7f, 0, 1.0f, 1.0f, 0},  {1.3f, 0, 1.0f, 1.0f, 0},
        {1.0f, 1, 1.0f, 1.0f, 0},  {1.0f, 5, 1.0f, 1.0f, 0},  {0.7f, 12, 1.0f, 1.0f, 0},
        {1.0f, 0, 0.9f, 1.0f, 0},  {1.0f, 0, 0.5f, 1.0f, 0},  {1.3f, 0, 0.2f, 1.0f, 0},
        {1.0f, 8, 0.7f, 1.0f, 0},  {0.8f, 0, 1.0f, 1.5f, 8},  {0.8f, 6, 0.8f, 2.0f, 10},
        {1.0f, 70, 1.0f, 1.0f, 0},
    };
    const int n_cases = (int)(sizeof(cases) / sizeof(cases[0]));
    Sampler sampler;
    std::printf("{\"vocab\": %d, \"draws\": %d, \"cases\": [\n", vocab, draws);
    for (int c = 0; c < n_cases; ++c) {
        lcg_state = 12345u + 977u * (uint32_t)c;
        std::vector<float> logits(vocab);
        for (float& v : logits) v = next_logit();
        std::vector<int32_t> prev;
        for (int i = 0; i < cases[c].n_prev; ++i) prev.push_back((int32_t)((7 * i + 3 * c) % vocab));
        SamplingParams p;
        p.temperature = cases[c].temperature;
        p.top_k = cases[c].top_k;
        p.top_p = cases[c].top_p;
        p.repetition_penalty = cases[c].penalty;
        std::vector<int> hist(vocab, 0);
        const int n = p.temperature == 0.0f ? 1 : draws;
        for (int i = 0; i < n; ++i) hist[sampler.sample(logits.data(), vocab, p, prev)]++;
        std::printf("  {\"case\": %d, \"temperature\": %.9g, \"top_k\": %d, \"top_p\": %.9g, "
                    "\"repetition_penalty\": %.9g, \"n_prev\": %d, \"draws\": %d, \"hist\": [",
                    c, p.temperature, p.top_k, p.top_p, p.repetition_penalty, cases[c].n_prev, n);
        for (int i = 0; i < vocab; ++i) std::printf("%d%s", hist[i], i + 1 < vocab ? ", " : "");
        std::printf("]}%s\n", c + 1 < n_cases ? "," : "");
    }
    std::printf("]}\n");
    return 0;
}
