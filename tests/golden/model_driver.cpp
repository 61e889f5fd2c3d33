// Drives the reference's own Llama model (models/llama/llama_model.cpp behind
// models/include/models/model_interface.h) through its public prefill()/decode() calls and
// writes the logits it returns, so that the plain implementation under tests/ can be held to
// them.  Built and run by make_model_golden.py on a machine with a GPU; nothing of the engine is
// linked in, and nothing of this file is part of the engine.
//
// usage: model_driver <model folder> <output file>     commands on standard input:
//   prefill N                     then N lines:  <start_pos> <n_tokens> <n_blocks> blocks... tokens...
//   decode N                      then N lines:  <seq_len> <n_blocks> blocks... <new token>
// Each command appends N rows of vocab floats (little-endian 32-bit) to the output file: for a
// prefill the logits of each request's last token, for a decode those of each new token
// (ForwardResult, model_interface.h:42-45).
#include <cstdio>
#include <iostream>
#include <memory>
#include <string>
#include <vector>

#include "kernels/cublas_provider.h"
#include "models/model_interface.h"

std::unique_ptr<ModelModule> create_llama_model(KernelProvider* kernels);

int main(int argc, char** argv) {
    if (argc != 3) {
        std::fprintf(stderr, "usage: %s <model folder> <output file>\n", argv[0]);
        return 2;
    }
    CublasProvider provider;
    std::unique_ptr<ModelModule> model = create_llama_model(&provider);
    model->load_weights(argv[1]);
    std::FILE* out = std::fopen(argv[2], "wb");
    if (!out) return 3;
    cudaStream_t stream;
    if (cudaStreamCreate(&stream) != cudaSuccess) return 4;
    std::string cmd;
    int n = 0;
    long rows = 0;
    while (std::cin >> cmd >> n) {
        const bool prefill = cmd == "prefill";
        if (!prefill && cmd != "decode") return 5;
        std::vector<RequestContext> reqs(n);
        for (int r = 0; r < n; ++r) {
            RequestContext& rc = reqs[r];
            rc.request_id = r;
            rc.max_new_tokens = 1;
            int n_blocks = 0;
            if (prefill) {
                std::cin >> rc.prefill_start_pos >> rc.prefill_chunk_len >> n_blocks;
                rc.seq_len = rc.prefill_start_pos + rc.prefill_chunk_len;
            } else {
                std::cin >> rc.seq_len >> n_blocks;
                rc.prefill_start_pos = 0;
                rc.prefill_chunk_len = 0;
            }
            rc.block_table.resize(n_blocks);
            for (int& b : rc.block_table) std::cin >> b;
            rc.token_ids.resize(prefill ? rc.prefill_chunk_len : 1);
            for (int32_t& t : rc.token_ids) std::cin >> t;
        }
        if (!std::cin) return 6;
        ForwardResult res = prefill ? model->prefill(reqs, stream) : model->decode(reqs, stream);
        if (cudaStreamSynchronize(stream) != cudaSuccess || cudaGetLastError() != cudaSuccess) return 7;
        if ((long)res.logits.size() != (long)n * res.vocab_size) return 8;
        std::fwrite(res.logits.data(), sizeof(float), res.logits.size(), out);
        rows += n;
    }
    std::fclose(out);
    std::fprintf(stderr, "model_driver: %ld rows written\n", rows);
    return 0;
}
