// Exercises the C++ mirror of the reference's backend trait (include/larql_backend.hpp).
// usage: mirror_check <in.bin> <out.bin>
//   in : int32 rows, cols, top_k, batch; gate, up, down Q4_K bytes (rows * cols/256 * 144 each); x f32 [batch, cols]
//   out: f32 matvec [rows] of gate . x[0]; f32 walk out [batch, cols]; int32 count[batch]; uint32 hits (concatenated)
// Exit status 3 when no device / library is available (the mirror has no CPU fallback).
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "larql_backend.hpp"

static std::vector<uint8_t> read_all(const char* path) {
    std::vector<uint8_t> b;
    FILE* f = std::fopen(path, "rb");
    if (!f) return b;
    std::fseek(f, 0, SEEK_END);
    const long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    b.resize(n > 0 ? (size_t)n : 0);
    if (n > 0 && std::fread(b.data(), 1, b.size(), f) != b.size()) b.clear();
    std::fclose(f);
    return b;
}

int main(int argc, char** argv) {
    try {
        larql::CudaBackend be(0);
        if (argc < 3) {
            std::printf("%s %s\n", be.name().c_str(), be.device_info().c_str());
            return 0;
        }
        const std::vector<uint8_t> in = read_all(argv[1]);
        if (in.size() < 16) return 2;
        const int32_t* hdr = reinterpret_cast<const int32_t*>(in.data());
        const size_t rows = hdr[0], cols = hdr[1], top_k = hdr[2], batch = hdr[3];
        const size_t mat = rows * (cols / 256) * 144;
        const uint8_t* gate = in.data() + 16;
        const uint8_t* up = gate + mat;
        const uint8_t* down = up + mat;
        const float* x = reinterpret_cast<const float*>(down + mat);
        if (in.size() != 16 + 3 * mat + batch * cols * 4) return 2;

        if (!be.supports_quant(larql::QuantFormat::Q4_K) || !be.supports_quant(larql::QuantFormat::NVFP4)) return 4;
        // refusals are nullopt, as the trait's None: wrong x length, hidden not a multiple of 256
        if (be.q4k_matvec(gate, mat, x, cols - 1, rows, cols).has_value()) return 5;
        if (be.q4k_matvec(gate, mat, x, cols, rows, cols + 32).has_value()) return 5;
        auto mv = be.q4k_matvec(gate, mat, x, cols, rows, cols);
        if (!mv) return 6;
        larql::QuantMatrix g{larql::QuantFormat::Q4_K, gate, mat, nullptr, 0, 1.0f, (int64_t)rows, (int64_t)cols, false};
        larql::QuantMatrix u = g, d = g;
        u.data = up;
        d.data = down;
        auto wr = be.walk_ffn(g, u, d, x, batch, top_k, LQ_WALK_FORCE_SPARSE);
        if (!wr) return 7;
        FILE* f = std::fopen(argv[2], "wb");
        if (!f) return 8;
        std::fwrite(mv->data(), 4, mv->size(), f);
        std::fwrite(wr->out.data(), 4, wr->out.size(), f);
        for (size_t t = 0; t < batch; ++t) {
            const int32_t c = (int32_t)wr->hits[t].size();
            std::fwrite(&c, 4, 1, f);
        }
        for (size_t t = 0; t < batch; ++t) std::fwrite(wr->hits[t].data(), 4, wr->hits[t].size(), f);
        std::fclose(f);
        return 0;
    } catch (const larql::BackendError& e) {
        std::fprintf(stderr, "BackendError(%d): %s\n", e.status, e.what());
        return 3;
    }
}
