// Drives the reference's own CPU backend (built out of tree from its sources) over a model
// folder and writes logits: used once to anchor tests/plain/qwen3_plain.py.
//   ref_driver MODEL_DIR OUT.bin FIRST_BLOCK CHUNK tok tok tok ...
// Feeds the tokens in chunks of CHUNK (0 = whole) with the block table starting at
// FIRST_BLOCK and, after every chunk, appends the logits of the chunk's last token
// (float32 [vocab]) to OUT.bin.
//   ref_driver sample LOGITS.bin VOCAB CASES.txt OUT.txt
// Draws one token per case with the reference's host sampler (src/backend/sampling_host.cpp:68-85).  A case is
// a line "row temperature top_p top_k min_p seed counter"; LOGITS.bin holds float32 rows of VOCAB values.  OUT.txt
// gets, per case, the token and the number of tokens its sampling distribution keeps.
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "backend/backend.hpp"
#include "backend/sampling_host.hpp"
#include "model_helpers.hpp"

static int sample_mode(int argc, char** argv) {
    if (argc < 6) return 2;
    const int vocab = std::atoi(argv[3]);
    std::vector<float> logits;
    {
        FILE* f = std::fopen(argv[2], "rb");
        if (!f) return 3;
        float buf[4096];
        size_t n;
        while ((n = std::fread(buf, sizeof(float), 4096, f)) > 0) logits.insert(logits.end(), buf, buf + n);
        std::fclose(f);
    }
    FILE* cases = std::fopen(argv[4], "r");
    FILE* out = std::fopen(argv[5], "w");
    if (!cases || !out) return 3;
    int row, top_k;
    float temperature, top_p, min_p;
    unsigned long long seed, counter;
    while (std::fscanf(cases, "%d %f %f %d %f %llu %llu", &row, &temperature, &top_p, &top_k, &min_p, &seed, &counter) == 7) {
        ember::SampleRequest req;
        req.params.temperature = temperature;
        req.params.top_p = top_p;
        req.params.top_k = top_k;
        req.params.min_p = min_p;
        req.params.seed = seed;
        req.counter = counter;
        const float* x = logits.data() + static_cast<size_t>(row) * static_cast<size_t>(vocab);
        std::fprintf(out, "%d %zu\n", ember::sample_host(x, vocab, req), ember::sampling_distribution(x, vocab, req.params).size());
    }
    std::fclose(cases);
    std::fclose(out);
    return 0;
}

int main(int argc, char** argv) {
    if (argc >= 2 && std::string(argv[1]) == "sample") return sample_mode(argc, argv);
    if (argc < 6) return 2;
    std::string dir = argv[1], out = argv[2];
    int first_block = std::atoi(argv[3]), chunk = std::atoi(argv[4]);
    std::vector<int> toks;
    for (int i = 5; i < argc; i++) toks.push_back(std::atoi(argv[i]));
    ember::BackendOptions opt;
    opt.device = "cpu";
    opt.kv_cache_tokens = 1024;
    opt.threads = 2;
    auto be = ember::create_backend(dir, opt);
    ember::test::SingleSequence seq(*be, first_block);
    if (chunk <= 0) chunk = (int)toks.size();
    FILE* f = std::fopen(out.c_str(), "wb");
    std::vector<float> row((size_t)be->config().vocab_size);
    for (size_t s = 0; s < toks.size(); s += (size_t)chunk) {
        size_t e = std::min(toks.size(), s + (size_t)chunk);
        seq.step(std::vector<int>(toks.begin() + (long)s, toks.begin() + (long)e));
        be->logits(0, row);
        std::fwrite(row.data(), sizeof(float), row.size(), f);
    }
    std::fclose(f);
    return 0;
}
