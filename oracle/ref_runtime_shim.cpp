// ref_runtime_shim.cpp -- C-ABI doorway into the UNMODIFIED reference's model runtime, compiled from its own
// sources where they lie (see oracle/Makefile; nothing is copied).
//
// TEST INFRASTRUCTURE ONLY.  libzenrt.so exists to produce golden token ids and logits for a small generated
// GGUF model (tests/golden/make_llama_golden.py); the product never loads it.  The wrapper forwards to
// zen::runtime::load_model_runtime and ModelRuntime::generate (include/zen/model_runtime.h:14-39) and adds no
// arithmetic of its own.
#include "zen/model_runtime.h"

#include <cstring>
#include <string>
#include <vector>

extern "C" {

// Greedy generation (temperature 0, the default GenerationOptions).  Returns the number of generated ids, or a
// negative value with a message in `err`.
int zrt_generate(const char* gguf_path, const unsigned* prompt, unsigned prompt_len, unsigned max_new, unsigned* out_ids,
                 float* out_logits, unsigned logits_cap, char* err, unsigned err_cap) {
    std::string error;
    auto fail = [&](int code) {
        if (err && err_cap) { std::strncpy(err, error.c_str(), err_cap - 1); err[err_cap - 1] = 0; }
        return code;
    };
    auto model = zen::runtime::load_model_runtime(gguf_path, nullptr, &error);
    if (!model) return fail(-1);
    zen::runtime::Generation g;
    const std::vector<std::uint32_t> p(prompt, prompt + prompt_len);
    if (!model->generate(p, max_new, g, &error)) return fail(-2);
    for (std::size_t i = 0; i < g.token_ids.size() && i < max_new; ++i) out_ids[i] = g.token_ids[i];
    for (std::size_t i = 0; i < g.last_logits.size() && i < logits_cap; ++i) out_logits[i] = g.last_logits[i];
    return static_cast<int>(g.token_ids.size());
}

}  // extern "C"
