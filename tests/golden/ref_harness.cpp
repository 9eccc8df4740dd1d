// Drives the reference's own code (garana/locus: src/locus/model/llama.cpp and arch.cpp on its CPU
// backends).  Used by make_golden.py to produce tests/golden/golden.json and the timings beside it; it
// is not part of the product and is compiled against the reference tree only (its GGUF image builder
// comes from the reference's tests/gguf_builder.hpp).
//
//   ref_harness logits <model file>
//       the logits of every position of the file's tokens (LlamaModel::forward, scalar backend)
//   ref_harness time <model file> <backend> <n decode>
//       seconds of a batched prefill of the file's tokens (forward_batch) and of <n decode> greedy
//       decode steps (forward) on the named backend
//   ref_harness select <selection file>
//       the reference's moe_select (llama.cpp:900-980) on rows of router logits: per row k expert ids,
//       then k weights
//
// Model file: u32 n_u32 {str key, u32 value}, u32 n_f32 {str key, f32 value},
//             u32 n_tensors {str name, u32 ndims, u64 dims (fastest first), f32 data},
//             u32 n_tokens {i32 token};   str = u32 length + bytes.
// Selection file: u32 E, k, renorm, gating (1 softmax, 2 sigmoid), n_group, n_group_used, has_bias;
//             f32 scale; f32 bias[E] when has_bias; u32 n_rows; f32 logits[n_rows][E].
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

#include "gguf_builder.hpp"
#include "locus/backend/registry.hpp"
#include "locus/gguf/gguf.hpp"
#include "locus/kv/paged_cache.hpp"
#include "locus/model/llama.hpp"

template <typename T>
static T rd(std::ifstream& f) {
    T v;
    f.read(reinterpret_cast<char*>(&v), sizeof(T));
    return v;
}
static std::string rd_str(std::ifstream& f) {
    const auto n = rd<std::uint32_t>(f);
    std::string s(n, '\0');
    f.read(s.data(), n);
    return s;
}

static int run_select(const char* path) {
    std::ifstream f(path, std::ios::binary);
    locus::model::Hparams hp;
    hp.n_expert = rd<std::uint32_t>(f);
    hp.n_expert_used = rd<std::uint32_t>(f);
    hp.expert_weights_norm = rd<std::uint32_t>(f) != 0;
    hp.gating = static_cast<locus::model::GatingFunc>(rd<std::uint32_t>(f));
    hp.n_group = rd<std::uint32_t>(f);
    hp.n_group_used = rd<std::uint32_t>(f);
    const bool has_bias = rd<std::uint32_t>(f) != 0;
    hp.expert_weights_scale = rd<float>(f);
    std::vector<float> bias(has_bias ? hp.n_expert : 0);
    for (auto& v : bias) v = rd<float>(f);
    locus::model::LlamaModel::Layer lay;
    if (has_bias) lay.exp_probs_b = bias;
    const auto n_rows = rd<std::uint32_t>(f);
    std::vector<float> row(hp.n_expert);
    for (std::uint32_t r = 0; r < n_rows; ++r) {
        for (auto& v : row) v = rd<float>(f);
        const auto picks = locus::model::moe_select(hp, lay, row);
        for (const auto& p : picks) std::printf("%u ", p.first);
        for (const auto& p : picks) std::printf("%.9g ", p.second);
        std::printf("\n");
    }
    return 0;
}

int main(int argc, char** argv) {
    if (argc < 3) return 2;
    const std::string mode = argv[1];
    if (mode == "select") return run_select(argv[2]);
    std::ifstream f(argv[2], std::ios::binary);
    struct T {
        std::string name;
        std::vector<std::uint64_t> dims;
        std::vector<float> data;
    };
    std::vector<std::pair<std::string, std::uint32_t>> ku;
    std::vector<std::pair<std::string, float>> kf;
    for (auto n = rd<std::uint32_t>(f); n > 0; --n) {
        auto k = rd_str(f);
        ku.emplace_back(k, rd<std::uint32_t>(f));
    }
    for (auto n = rd<std::uint32_t>(f); n > 0; --n) {
        auto k = rd_str(f);
        kf.emplace_back(k, rd<float>(f));
    }
    std::vector<T> tensors;
    for (auto n = rd<std::uint32_t>(f); n > 0; --n) {
        T t;
        t.name = rd_str(f);
        const auto nd = rd<std::uint32_t>(f);
        std::size_t count = 1;
        for (std::uint32_t i = 0; i < nd; ++i) {
            t.dims.push_back(rd<std::uint64_t>(f));
            count *= t.dims.back();
        }
        t.data.resize(count);
        f.read(reinterpret_cast<char*>(t.data.data()), count * 4);
        tensors.push_back(std::move(t));
    }
    std::vector<std::int32_t> tokens;
    for (auto n = rd<std::uint32_t>(f); n > 0; --n) tokens.push_back(rd<std::int32_t>(f));

    GgufBuilder b;
    b.header(tensors.size(), 1 + ku.size() + kf.size()).kv_string("general.architecture", "qwen2moe");
    for (auto& [k, v] : ku) b.kv_u32(k, v);
    for (auto& [k, v] : kf) b.kv_f32(k, v);
    std::uint64_t offset = 0;
    for (const auto& t : tensors) {
        b.tensor(t.name, t.dims, 0 /* F32 */, offset);
        offset = (offset + t.data.size() * 4 + 31) & ~31ull;
    }
    b.pad();
    for (const auto& t : tensors) {
        for (float v : t.data) b.f32(v);
        b.pad();
    }
    auto span = b.bytes();
    std::vector<std::byte> image(span.begin(), span.end());

    auto g = locus::gguf::GgufFile::parse(image);
    auto model = locus::model::LlamaModel::load(g);
    if (mode == "time") {
        if (argc < 5) return 2;
        const auto* backend = locus::backend::find_backend(argv[3]);
        if (backend == nullptr) {
            std::printf("unavailable\n");
            return 0;
        }
        model.use_backend(*backend);
        const int n_decode = std::atoi(argv[4]);
        auto cache = model.make_cache();
        auto ws = model.make_workspace();
        locus::kv::PagedKvCache::Seq seq;
        std::vector<float> logits(model.hparams().n_vocab);
        using clock = std::chrono::steady_clock;
        if (!cache.ensure_capacity(seq, tokens.size() + n_decode)) return 3;
        const auto t0 = clock::now();
        if (model.supports_batch() && tokens.size() >= 2) {
            model.forward_batch(tokens, cache, seq, ws, logits);
        } else {
            for (auto t : tokens) model.forward(t, cache, seq, ws, logits);
        }
        const auto t1 = clock::now();
        for (int i = 0; i < n_decode; ++i) {
            const auto next = static_cast<std::int32_t>(locus::model::argmax(logits));
            model.forward(next, cache, seq, ws, logits);
        }
        const auto t2 = clock::now();
        std::printf("%zu %.6f %d %.6f\n", tokens.size(), std::chrono::duration<double>(t1 - t0).count(), n_decode,
                    std::chrono::duration<double>(t2 - t1).count());
        cache.release(seq);
        return 0;
    }
    model.use_backend(*locus::backend::find_backend("scalar"));
    auto cache = model.make_cache();
    auto ws = model.make_workspace();
    locus::kv::PagedKvCache::Seq seq;
    std::vector<float> logits(model.hparams().n_vocab);
    std::printf("%zu %u\n", tokens.size(), model.hparams().n_vocab);
    for (auto t : tokens) {
        if (!cache.ensure_capacity(seq, 1)) return 3;
        model.forward(t, cache, seq, ws, logits);
        for (float v : logits) std::printf("%.9g ", v);
        std::printf("\n");
    }
    cache.release(seq);
    return 0;
}
