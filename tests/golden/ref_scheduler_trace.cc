// Drives the reference's own scheduler (src/scheduler.cc, src/radix_tree.cc, compiled unchanged) through
// the bookkeeping its engine loop does (src/engine.cc:222-271 for prompt portions, :296-345 for decode
// tokens, :381-440 for finishing) and prints, per iteration, which request was fed how many tokens from
// which context length.  No model runs: every "generated" token is the constant 7.
#include <algorithm>
#include <cstdio>
#include <memory>
#include <string>
#include <vector>

#include "firefly/scheduler.h"

using namespace firefly;

int main(int argc, char** argv) {
    if (argc < 5 || (argc - 4) % 3 != 0) {
        std::fprintf(stderr, "usage: %s BLOCKS MAX_BATCH CHUNK (ID PROMPT_LEN MAX_TOKENS)...\n", argv[0]);
        return 2;
    }
    const int blocks = std::atoi(argv[1]), max_batch = std::atoi(argv[2]), chunk = std::atoi(argv[3]);
    Scheduler sched;
    sched.init(blocks, max_batch, chunk);
    int next_token = 100;                       // distinct prompts: no prefix is shared
    for (int a = 4; a + 2 < argc; a += 3) {
        std::vector<int> prompt(std::atoi(argv[a + 1]));
        for (int& t : prompt) t = next_token++;
        sched.add_request(std::make_shared<GenerationRequest>(argv[a], prompt, std::atoi(argv[a + 2])));
    }
    std::printf("[");
    bool first_step = true;
    for (int iter = 0; iter < 1000 && sched.has_unfinished_requests(); ++iter) {
        SchedulerBatch batch = sched.step();
        if (batch.requests.empty()) break;      // the reference would spin here
        std::vector<RequestPtr> prefill, decode;
        for (auto& r : batch.requests) (r->generated_tokens.empty() ? prefill : decode).push_back(r);
        std::printf("%s[", first_step ? "" : ",\n ");
        first_step = false;
        bool first = true;
        auto emit = [&](const RequestPtr& r, int n) {
            std::printf("%s[\"%s\", %d, %d, %d]", first ? "" : ", ", r->id.c_str(), r->context_len, n,
                        (int)r->block_table.size());
            first = false;
        };
        for (auto& r : batch.requests) {        // in the batch's order
            if (std::find(prefill.begin(), prefill.end(), r) != prefill.end()) {
                const int n = std::min((int)r->prompt_tokens.size() - r->context_len, chunk);
                emit(r, n);
                r->context_len += n;
                if (r->context_len == (int)r->prompt_tokens.size()) r->generated_tokens.push_back(7);
            } else {
                emit(r, 1);
                r->context_len += 1;
                r->generated_tokens.push_back(7);
            }
        }
        std::printf("]");
        for (auto& r : batch.requests)
            if (!r->generated_tokens.empty() && (int)r->generated_tokens.size() >= r->max_tokens)
                sched.finish_request(r);
    }
    std::printf("]\n");
    return 0;
}
