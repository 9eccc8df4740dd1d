// Drives the reference's own model code (garana/locus, src/locus/model/llama.cpp and arch.cpp,
// scalar CPU backend) on a model given as a flat binary file, and prints the logits of every
// position.  Used once by make_golden.py to produce tests/golden/golden.json; it is not part
// of the product and is compiled against the reference tree only (its GGUF image builder comes
// from the reference's tests/gguf_builder.hpp).
//
// Input file: u32 n_u32 {str key, u32 value}, u32 n_f32 {str key, f32 value},
//             u32 n_tensors {str name, u32 ndims, u64 dims (fastest first), f32 data},
//             u32 n_tokens {i32 token};   str = u32 length + bytes.
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

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    std::ifstream f(argv[1], std::ios::binary);
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
