// Driver of tests/test_loader.py for include/strata_moe_loader.hpp.
//   list <file.safetensors>                          name dtype shape bytes fnv1a64 per tensor
//   untile <hidden> <intermediate> <out> <shard>...  canonical tensors rebuilt from tiled shards -> <out>.{w1,s1,w3,s3,w2,s2}
//   trace <out.jsonl>                                a fixed page of routes as strata.route_trace v2
//   forward <file> <family> <layer> <fmt> <H> <I> <E> <k> <Is> <score> <x.bin> <T> <out.bin>
//                                                    load the layer from the checkpoint, run it on x (needs a GPU)
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "strata_moe_loader.hpp"

using namespace strata_b200;

static std::vector<std::byte> slurp(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    std::vector<char> c((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    std::vector<std::byte> b(c.size());
    if (!c.empty()) std::memcpy(b.data(), c.data(), c.size());   // an empty file has no storage to copy from
    return b;
}
static void dump(const std::string& path, const void* p, std::size_t n) {
    std::ofstream f(path, std::ios::binary);
    f.write(static_cast<const char*>(p), static_cast<std::streamsize>(n));
}
static int report(const LoadResult& r) {
    for (const auto& e : r.errors) std::fprintf(stderr, "error: %s\n", e.c_str());
    return r.ok() ? 0 : 1;
}

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    const std::string cmd = argv[1];
    if (cmd == "list" && argc == 3) {
        SafetensorsFile f;
        if (report(f.open(argv[2]))) return 1;
        for (const auto& [name, t] : f.tensors()) {
            std::uint64_t h = 1469598103934665603ULL;
            for (std::size_t i = 0; i < t.bytes; ++i) h = (h ^ static_cast<std::uint8_t>(t.data[i])) * 1099511628211ULL;
            std::printf("%s %s ", name.c_str(), t.dtype.c_str());
            for (std::size_t i = 0; i < t.shape.size(); ++i) std::printf("%s%llu", i ? "x" : "", (unsigned long long)t.shape[i]);
            std::printf(" %zu %016llx\n", t.bytes, (unsigned long long)h);
        }
        return 0;
    }
    if (cmd == "untile" && argc >= 6) {
        const std::uint64_t H = std::strtoull(argv[2], nullptr, 10), I = std::strtoull(argv[3], nullptr, 10);
        std::vector<std::vector<std::byte>> storage;
        for (int i = 5; i < argc; ++i) storage.push_back(slurp(argv[i]));
        std::vector<std::span<const std::byte>> views(storage.begin(), storage.end());
        CanonicalExpert e;
        if (report(tiled32_to_canonical(views, H, I, e))) return 1;
        const std::string out = argv[4];
        dump(out + ".w1", e.w1.data(), e.w1.size());
        dump(out + ".s1", e.s1.data(), e.s1.size());
        dump(out + ".w3", e.w3.data(), e.w3.size());
        dump(out + ".s3", e.s3.data(), e.s3.size());
        dump(out + ".w2", e.w2.data(), e.w2.size());
        dump(out + ".s2", e.s2.data(), e.s2.size());
        return 0;
    }
    if (cmd == "trace" && argc == 3) {
        RouteTraceWriter w;
        if (report(w.open(argv[2]))) return 1;
        const std::vector<std::uint32_t> ids{5, 1, 7, 2, 0, 3};
        const std::vector<float> weights{0.5F, 0.25F, 0.125F, 0.3333333F, 1.0e-7F, 0.6666666F};
        if (report(w.write_page(42, RoutePhase::Prefill, 10, 3, ids, weights, 3))) return 1;
        RouteEvent e;
        e.request = 43;
        e.phase = RoutePhase::Decode;
        e.token_position = 99;
        e.layer = 7;
        e.experts = {11};
        if (report(w.write(e))) return 1;          // coefficients may be absent
        e.coefficients = {1.0F, 2.0F};
        if (w.write(e).ok()) return 1;             // mismatched coefficient count is refused
        w.close();
        return 0;
    }
    if (cmd == "forward" && argc == 15) {
        SafetensorsFile f;
        if (report(f.open(argv[2]))) return 1;
        const std::string fam = argv[3];
        const MoeFamily family = fam == "dsv4" ? MoeFamily::DeepSeekV4 : fam == "glm" ? MoeFamily::Glm
                                 : fam == "laguna" ? MoeFamily::Laguna : MoeFamily::KimiK3;
        strata_moe_layer_desc d{};
        const std::uint32_t layer_index = static_cast<std::uint32_t>(std::atoi(argv[4]));
        d.format = std::atoi(argv[5]);
        d.hidden = static_cast<std::uint32_t>(std::atoi(argv[6]));
        d.intermediate = static_cast<std::uint32_t>(std::atoi(argv[7]));
        d.experts = d.expert_count = static_cast<std::uint32_t>(std::atoi(argv[8]));
        d.top_k = static_cast<std::uint32_t>(std::atoi(argv[9]));
        d.shared_intermediate = static_cast<std::uint32_t>(std::atoi(argv[10]));
        d.score_kind = std::atoi(argv[11]);
        d.normalize = 1;
        d.weight_scale = d.output_scale = 1.0F;
        const std::uint32_t T = static_cast<std::uint32_t>(std::atoi(argv[13]));
        d.max_tokens = T;
        strata_moe_ctx* ctx = nullptr;
        if (strata_moe_create(0, nullptr, &ctx) != 0) { std::fprintf(stderr, "no usable device\n"); return 3; }
        strata_moe_layer* layer = nullptr;
        if (strata_moe_layer_create(ctx, &d, &layer) != 0) { std::fprintf(stderr, "%s\n", strata_moe_last_error(ctx)); return 1; }
        const SafetensorsFile* files[1] = {&f};
        if (report(load_moe_layer(layer, d, files, family, layer_index))) return 1;
        const auto x = slurp(argv[12]);
        std::vector<float> out(static_cast<std::size_t>(T) * d.hidden);
        if (strata_moe_forward_host(layer, x.data(), T, out.data()) != 0) { std::fprintf(stderr, "%s\n", strata_moe_last_error(ctx)); return 1; }
        dump(argv[14], out.data(), out.size() * 4);
        strata_moe_layer_destroy(layer);
        strata_moe_destroy(ctx);
        return 0;
    }
    return 2;
}
