// Runs celsowm/celeg's own CPU model (celeg::CpuModel, its default 4-bit group-32 weights) on a model
// folder and a fixed prompt and prints the logits of the last prompt token as JSON. Built and run by
// make_golden_model.sh against the reference checkout and its library; the result is committed as
// golden_model.json and compared by tests/test_golden_reference.py with the plain implementation after the
// reference's two known artefacts (4-bit weights, attention scores scaled twice) have been emulated there.
#include "celeg/backend/cpu/model.hpp"

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

int main(int argc, char** argv) {
    if (argc < 3) {
        std::fprintf(stderr, "usage: %s MODEL_DIR TOKEN [TOKEN ...]\n", argv[0]);
        return 2;
    }
    std::vector<int32_t> prompt;
    for (int i = 2; i < argc; ++i) prompt.push_back(std::atoi(argv[i]));
    celeg::CpuModelOptions options;
    options.use_pack_cache = false;
    options.threads = 1;
    options.kv_cache_mode = celeg::CpuKvCacheMode::Fp32;
    celeg::CpuModel model(argv[1], 256, options);
    model.session().prefill(prompt);
    const std::vector<float> logits = model.diagnostics().copy_logits();
    std::printf("{\n  \"backend\": \"%s\",\n  \"prompt\": [", model.diagnostics().backend_description().c_str());
    for (size_t i = 0; i < prompt.size(); ++i) std::printf("%s%d", i ? "," : "", prompt[i]);
    std::printf("],\n  \"logits_last\": [");
    for (size_t i = 0; i < logits.size(); ++i) std::printf("%s%.9g", i ? "," : "", logits[i]);
    std::printf("]\n}\n");
    return 0;
}
