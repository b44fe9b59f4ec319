// Readers for the on-disk K-quant FFN weights of a vindex directory (host code, no device work):
//   interleaved_kquant.bin + interleaved_kquant_manifest.json   per layer [gate Q4_K | up Q4_K | down Q4_K/Q6_K],
//       written by write_interleaved_ffn_kquant
//       (crates/larql-vindex/src/format/weights/write_kquant/ffn.rs:25-117);
//   down_features_kquant.bin + down_features_kquant_manifest.json   the down weights transposed to
//       feature-major [padded intermediate, padded hidden]
//       (crates/larql-vindex/src/format/weights/write_kquant/feature_major_down.rs:48-104);
//   the legacy names interleaved_q4k.bin / down_features_q4k.bin with their manifests
//       (crates/larql-vindex/src/format/filenames.rs:80-97).
// A manifest is a JSON array of {key, shape [rows, padded cols], format "Q4_K" | "Q6_K", offset, length}
// (Q4kManifestEntry, crates/larql-vindex/src/format/weights/manifest.rs:23-31), three entries per layer in
// gate, up, down order (load_interleaved_kquant / interleaved_kquant_layer_data,
// crates/larql-vindex/src/index/storage/ffn_store/interleaved_kquant.rs:64-190).  Every row is padded to a
// whole number of 256-element super-blocks (k_quant_padded_cols,
// crates/larql-models/src/quant/ggml/mod.rs:105-114); readers index rows at the padded stride.
// Also: the three regions of a stored NVFP4 tensor (PackLayout::derive / split,
// crates/larql-vindex/src/format/vindex3/represent/nvfp4_pack.rs).
// The files are mapped read-only and demand-paged, as the reference does; the matrices handed out point into
// the mappings and stay valid until lq_vindex_close.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/larql_cuda.h"

namespace {

struct Entry {
    std::string key, format;
    std::vector<long long> shape;
    long long offset = -1, length = -1;
};

struct Mapped {
    const uint8_t* p = nullptr;
    size_t len = 0;
    bool open_ro(const std::string& path, std::string& err) {
        const int fd = ::open(path.c_str(), O_RDONLY);
        if (fd < 0) {
            err = path + ": cannot open";
            return false;
        }
        struct stat st;
        if (fstat(fd, &st) != 0) {
            ::close(fd);
            err = path + ": cannot stat";
            return false;
        }
        len = (size_t)st.st_size;
        if (len > 0) {
            void* m = mmap(nullptr, len, PROT_READ, MAP_PRIVATE, fd, 0);
            if (m == MAP_FAILED) {
                ::close(fd);
                err = path + ": mmap failed";
                return false;
            }
            p = (const uint8_t*)m;
        }
        ::close(fd);
        return true;
    }
    void unmap() {
        if (p) munmap((void*)p, len);
        p = nullptr;
        len = 0;
    }
};

bool file_exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

bool read_text(const std::string& path, std::string& out) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    char buf[65536];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) out.append(buf, n);
    fclose(f);
    return true;
}

// A small JSON reader for the manifest's shape: an array of flat objects whose values are strings, integers
// or arrays of integers.  Anything else is a parse error (a renamed or retyped field fails loudly).
struct Json {
    const std::string& s;
    size_t i = 0;
    std::string err;
    explicit Json(const std::string& t) : s(t) {}
    void ws() {
        while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i;
    }
    bool eat(char c) {
        ws();
        if (i < s.size() && s[i] == c) {
            ++i;
            return true;
        }
        return false;
    }
    bool str(std::string& out) {
        ws();
        if (i >= s.size() || s[i] != '"') return false;
        ++i;
        out.clear();
        while (i < s.size() && s[i] != '"') {
            if (s[i] == '\\') {
                if (i + 1 >= s.size()) return false;
                const char e = s[i + 1];
                if (e == 'u') {  // keys and tags are ASCII; keep the escape as it is
                    out += "\\u";
                    i += 2;
                    continue;
                }
                out += (e == 'n' ? '\n' : e == 't' ? '\t' : e);
                i += 2;
            } else
                out += s[i++];
        }
        if (i >= s.size()) return false;
        ++i;
        return true;
    }
    bool integer(long long& v) {
        ws();
        const size_t b = i;
        if (i < s.size() && s[i] == '-') ++i;
        while (i < s.size() && s[i] >= '0' && s[i] <= '9') ++i;
        if (i == b || (i == b + 1 && s[b] == '-')) return false;
        if (i < s.size() && (s[i] == '.' || s[i] == 'e' || s[i] == 'E')) return false;  // offsets are integers
        v = strtoll(s.c_str() + b, nullptr, 10);
        return true;
    }
    bool entries(std::vector<Entry>& out) {
        if (!eat('[')) return fail("manifest is not a JSON array");
        if (eat(']')) return true;
        do {
            Entry e;
            if (!eat('{')) return fail("manifest entry is not an object");
            if (!eat('}')) {
                do {
                    std::string k;
                    if (!str(k) || !eat(':')) return fail("bad key");
                    if (k == "key") {
                        if (!str(e.key)) return fail("key: expected a string");
                    } else if (k == "format") {
                        if (!str(e.format)) return fail("format: expected a string");
                    } else if (k == "offset") {
                        if (!integer(e.offset)) return fail("offset: expected an integer");
                    } else if (k == "length") {
                        if (!integer(e.length)) return fail("length: expected an integer");
                    } else if (k == "shape") {
                        if (!eat('[')) return fail("shape: expected an array");
                        if (!eat(']')) {
                            do {
                                long long v;
                                if (!integer(v)) return fail("shape: expected integers");
                                e.shape.push_back(v);
                            } while (eat(','));
                            if (!eat(']')) return fail("shape: unterminated array");
                        }
                    } else
                        return fail("unknown field `" + k + "`");
                } while (eat(','));
                if (!eat('}')) return fail("unterminated object");
            }
            if (e.offset < 0 || e.length < 0 || e.format.empty()) return fail("entry lacks offset, length or format");
            out.push_back(e);
        } while (eat(','));
        if (!eat(']')) return fail("unterminated array");
        return true;
    }
    bool fail(const std::string& m) {
        err = m;
        return false;
    }
};

int format_of(const std::string& tag) {  // the formats the reference's registry knows (quant/registry.rs)
    if (tag == "Q4_K") return LQ_FMT_Q4_K;
    if (tag == "Q6_K") return LQ_FMT_Q6_K;
    return -1;
}
size_t block_bytes(int fmt) { return fmt == LQ_FMT_Q4_K ? 144 : 210; }

bool load_manifest(const std::string& path, const Mapped& bin, std::vector<Entry>& out, std::string& err) {
    std::string text;
    if (!read_text(path, text)) {
        err = path + ": cannot read";
        return false;
    }
    Json j(text);
    if (!j.entries(out)) {
        err = path + ": " + j.err;
        return false;
    }
    for (size_t i = 0; i < out.size(); ++i) {
        const Entry& e = out[i];
        const int fmt = format_of(e.format);
        if (fmt < 0) {
            err = path + ": unknown format tag \"" + e.format + "\"";
            return false;
        }
        if (e.shape.size() < 2 || e.shape[0] < 0 || e.shape[1] < 0 || e.shape[1] % 256 != 0) {
            err = path + ": entry " + std::to_string(i) + " needs shape [rows, cols padded to 256]";
            return false;
        }
        const size_t need = (size_t)e.shape[0] * (size_t)(e.shape[1] / 256) * block_bytes(fmt);
        if ((size_t)e.length != need) {
            err = path + ": entry " + std::to_string(i) + " length does not match its shape and format";
            return false;
        }
        if ((size_t)e.offset + (size_t)e.length > bin.len) {
            err = path + ": entry " + std::to_string(i) + " reaches past the end of the weights file";
            return false;
        }
    }
    return true;
}

void matrix_of(const Entry& e, const Mapped& bin, lq_matrix* m) {
    m->fmt = format_of(e.format);
    m->data = bin.p + e.offset;
    m->data_len = (size_t)e.length;
    m->scales = nullptr;
    m->scales_len = 0;
    m->tensor_scale = 1.0f;
    m->rows = e.shape[0];
    m->cols = e.shape[1];
}

void put_err(char* err, size_t cap, const std::string& m) {
    if (err && cap) snprintf(err, cap, "%s", m.c_str());
}

}  // namespace

struct lq_vindex {
    Mapped ffn, down_fm;
    std::vector<Entry> ffn_entries, down_entries;
};

extern "C" {

size_t lq_k_quant_padded_cols(size_t cols) { return (cols + 255) / 256 * 256; }

int lq_vindex_open(const char* dir, lq_vindex** out, char* err, size_t err_cap) {
    if (!dir || !out) return LQ_ERR_ARGUMENT;
    *out = nullptr;
    const std::string d(dir);
    std::string bin = d + "/interleaved_kquant.bin", man = d + "/interleaved_kquant_manifest.json";
    if (!file_exists(bin)) {
        bin = d + "/interleaved_q4k.bin";
        man = d + "/interleaved_q4k_manifest.json";
    }
    if (!file_exists(bin)) {
        put_err(err, err_cap, "interleaved k-quant FFN not found (looked for interleaved_kquant.bin and legacy interleaved_q4k.bin)");
        return LQ_REFUSED_UNSUPPORTED;
    }
    lq_vindex* v = new lq_vindex();
    std::string e;
    if (!v->ffn.open_ro(bin, e)) {
        put_err(err, err_cap, e);
        delete v;
        return LQ_ERR_ARGUMENT;
    }
    if (!file_exists(man)) {
        // (vindexes without a manifest use one uniform Q4_K stride and need the shapes from index.json)
        put_err(err, err_cap, man + ": manifest missing");
        v->ffn.unmap();
        delete v;
        return LQ_REFUSED_UNSUPPORTED;
    }
    if (!load_manifest(man, v->ffn, v->ffn_entries, e) || v->ffn_entries.size() % 3 != 0) {
        put_err(err, err_cap, e.empty() ? man + ": not three entries (gate, up, down) per layer" : e);
        v->ffn.unmap();
        delete v;
        return LQ_REFUSED_SHAPE;
    }
    // feature-major down: optional, but a weights file without its manifest is an error
    std::string dbin = d + "/down_features_kquant.bin", dman = d + "/down_features_kquant_manifest.json";
    if (!file_exists(dbin)) {
        dbin = d + "/down_features_q4k.bin";
        dman = d + "/down_features_q4k_manifest.json";
    }
    if (file_exists(dbin)) {
        bool ok = file_exists(dman);
        if (!ok) e = dbin + " present but manifest " + dman + " missing";
        ok = ok && v->down_fm.open_ro(dbin, e) && load_manifest(dman, v->down_fm, v->down_entries, e);
        if (ok && v->down_entries.size() != v->ffn_entries.size() / 3) {
            ok = false;
            e = dman + ": one entry per layer expected";
        }
        if (!ok) {
            put_err(err, err_cap, e);
            v->ffn.unmap();
            v->down_fm.unmap();
            delete v;
            return LQ_REFUSED_SHAPE;
        }
    }
    *out = v;
    return LQ_OK;
}

size_t lq_vindex_num_layers(const lq_vindex* v) { return v ? v->ffn_entries.size() / 3 : 0; }

int lq_vindex_layer(const lq_vindex* v, size_t layer, lq_matrix* gate, lq_matrix* up, lq_matrix* down, lq_matrix* down_fm) {
    if (!v || layer >= v->ffn_entries.size() / 3) return LQ_ERR_ARGUMENT;
    if (gate) matrix_of(v->ffn_entries[3 * layer], v->ffn, gate);
    if (up) matrix_of(v->ffn_entries[3 * layer + 1], v->ffn, up);
    if (down) matrix_of(v->ffn_entries[3 * layer + 2], v->ffn, down);
    if (down_fm) {
        if (v->down_entries.empty()) {
            memset(down_fm, 0, sizeof *down_fm);
            down_fm->fmt = -1;  // no feature-major sidecar: the caller transposes `down`
        } else
            matrix_of(v->down_entries[layer], v->down_fm, down_fm);
    }
    return LQ_OK;
}

void lq_vindex_close(lq_vindex* v) {
    if (!v) return;
    v->ffn.unmap();
    v->down_fm.unmap();
    delete v;
}

int lq_nvfp4_pack_split(const uint8_t* bytes, size_t len, size_t rows, size_t k, lq_matrix* out) {
    if (!out || (!bytes && len)) return LQ_ERR_ARGUMENT;
    if (k % 16 != 0) return LQ_REFUSED_SHAPE;  // refuses rather than pads, as the encoder does
    const size_t groups = k / 16, packed_len = rows * groups * 8, scales_len = rows * groups;
    if (len != packed_len + scales_len + 4) return LQ_REFUSED_SHAPE;
    out->fmt = LQ_FMT_NVFP4;
    out->data = bytes;
    out->data_len = packed_len;
    out->scales = bytes + packed_len;
    out->scales_len = scales_len;
    memcpy(&out->tensor_scale, bytes + packed_len + scales_len, 4);  // little-endian f32
    out->rows = (int64_t)rows;
    out->cols = (int64_t)k;
    return LQ_OK;
}

}  // extern "C"
