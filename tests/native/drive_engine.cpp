// A C++ program that generates through the native engine's header alone (no Python in the process).
//
//   drive_engine MODEL_DIR KERNEL_DIR PAGE_SIZE   < requests
//
// MODEL_DIR holds config.json and model.safetensors; KERNEL_DIR the built kernel libraries.  Every line of standard
// input is one request: `greedy` or `seeded`, then the prompt's token ids.  The program loads the model in float32
// (`llmx::Engine::load`), adds the requests, steps until the engine is idle (two requests run at once, sixteen tokens
// a step, so prompts are cut and requests wait), and prints each reply's token ids on a line, in the requests' order.
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "llmx_engine.h"

int main(int argc, char** argv) {
    if (argc != 4) {
        fprintf(stderr, "usage: drive_engine MODEL_DIR KERNEL_DIR PAGE_SIZE\n");
        return 2;
    }
    try {
        llmx_engine_options opt = {};
        opt.dtype = LLMX_DT_F32;
        opt.kv_dtype = -1;
        opt.page_size = atoi(argv[3]);
        opt.kv_tokens = 512;
        opt.max_requests = 2;
        opt.max_batch_tokens = 16;
        opt.kernel_dir = argv[2];
        llmx::Engine engine = llmx::Engine::load(argv[1], opt);
        std::vector<long long> ids;
        std::string line;
        while (std::getline(std::cin, line)) {
            std::istringstream in(line);
            std::string kind;
            if (!(in >> kind)) continue;
            std::vector<int> prompt;
            for (int t; in >> t;) prompt.push_back(t);
            llmx_sampling s;
            if (kind == "greedy") {
                llmx_sampling_greedy(&s, 8);
            } else {
                llmx_sampling_defaults(&s);
                s.max_tokens = 8, s.temp = 0.9f, s.top_k = 10, s.top_p = 0.9f, s.seed = 5;
            }
            s.ignore_eos = 1;
            ids.push_back(engine.add_request(prompt, s));
        }
        long long steps = 0;
        while (!engine.idle()) {
            engine.step();
            if (++steps > 100000) {
                fprintf(stderr, "the engine does not become idle\n");
                return 1;
            }
        }
        for (long long id : ids) {
            int finished = 0;
            const std::vector<int> reply = engine.output(id, &finished);
            for (size_t i = 0; i < reply.size(); ++i) printf("%s%d", i ? " " : "", reply[i]);
            printf("\n");
            if (finished != 2) {
                fprintf(stderr, "request %lld ended with reason %d, not at its max_tokens\n", id, finished);
                return 1;
            }
        }
        if (llmx_engine_check(engine.get())) {
            fprintf(stderr, "cache: %s\n", llmx_engine_last_error());
            return 1;
        }
    } catch (const llmx::Error& e) {
        fprintf(stderr, "error %d: %s\n", e.code, e.what);
        return 1;
    }
    return 0;
}
