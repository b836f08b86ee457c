// cuda_runtime_shim.cpp -- C-ABI doorway into the reference's model runtime BUILT WITH THE CUDA BACKEND HOOKED IN
// (tests/integration/Makefile): load_model_runtime + ModelRuntime::generate (include/zen/model_runtime.h:14-39), then the
// backend's own counters, so the test can see that every projection went through libzen_cuda.so.
//
// TEST INFRASTRUCTURE ONLY; adds no arithmetic of its own.
#include "zen/cuda_backend.h"
#include "zen/model_runtime.h"

#include <cstring>
#include <string>
#include <vector>

extern "C" {

// Greedy generation.  Returns the number of generated ids, or a negative value with a message in `err`.  stats_out receives
// {submits, dispatches, fallbacks, upload_bytes} of the CUDA backend after the run; the backend is shut down before returning,
// which releases every tensor that was made resident from the file mapping.
int zrt_cuda_generate(const char* gguf_path, const unsigned* prompt, unsigned prompt_len, unsigned max_new, unsigned* out_ids,
                      float* out_logits, unsigned logits_cap, unsigned long long* stats_out, char* err, unsigned err_cap) {
    std::string error;
    auto fail = [&](int code) {
        if (error.empty()) error = zen::cuda::last_error();
        if (err && err_cap) { std::strncpy(err, error.c_str(), err_cap - 1); err[err_cap - 1] = 0; }
        zen::cuda::shutdown();
        return code;
    };
    if (!zen::cuda::enabled()) return fail(-3);
    int n = 0;
    {
        auto model = zen::runtime::load_model_runtime(gguf_path, nullptr, &error);
        if (!model) return fail(-1);
        zen::runtime::Generation g;
        const std::vector<std::uint32_t> p(prompt, prompt + prompt_len);
        if (!model->generate(p, max_new, g, &error)) return fail(-2);
        for (std::size_t i = 0; i < g.token_ids.size() && i < max_new; ++i) out_ids[i] = g.token_ids[i];
        for (std::size_t i = 0; i < g.last_logits.size() && i < logits_cap; ++i) out_logits[i] = g.last_logits[i];
        n = static_cast<int>(g.token_ids.size());
        const zen::cuda::Stats s = zen::cuda::stats();
        if (stats_out) { stats_out[0] = s.submits; stats_out[1] = s.dispatches; stats_out[2] = s.fallbacks; stats_out[3] = s.upload_bytes; }
        zen::cuda::shutdown();   // before the model (and its file mapping) goes: resident copies are keyed by addresses inside it
    }
    return n;
}

}  // extern "C"
