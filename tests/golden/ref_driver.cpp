// Drives the reference's own CPU backend (built out of tree from its sources) over a model
// folder and writes logits: used once to anchor tests/plain/qwen3_plain.py.
//   ref_driver MODEL_DIR OUT.bin FIRST_BLOCK CHUNK tok tok tok ...
// Feeds the tokens in chunks of CHUNK (0 = whole) with the block table starting at
// FIRST_BLOCK and, after every chunk, appends the logits of the chunk's last token
// (float32 [vocab]) to OUT.bin.
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "backend/backend.hpp"
#include "model_helpers.hpp"

int main(int argc, char** argv) {
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
