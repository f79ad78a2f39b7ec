// On-disk formats either side of the sparse front end: the reference's weight files (".wts") with what the
// network builder does to the numbers before the sparse layers see them, and its point cloud files.
// Host code only.
//
// File format, as written by the reference's exporter (tools/gen_wts.py:85-99) and read by loadWeights
// (se-ssd-ai-trt.cpp:278-314): the first token is the number of blobs in decimal; every blob is
// `name count` followed by `count` words of eight hex digits, each the IEEE-754 bit pattern of one fp32
// value (the exporter prints the big-endian bytes, which read back as the plain hexadecimal number).
// Tokens are separated by any white space. A SubM / SpConv weight blob is the flattened
// [k0][k1][k2][Cin][Cout] tensor, which is the [kvol][Cin][Cout] layout the conv entry points take.
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "sessd.h"

struct sessd_wts {
    std::vector<std::string> names;
    std::vector<std::vector<float>> values;
    std::unordered_map<std::string, int> index;   // a repeated name keeps the last blob, like the reference's map
};

namespace {

// Walks white-space separated tokens of a buffer held in memory.
struct Tokens {
    const char* p;
    const char* end;
    bool next(const char** tok, size_t* len) {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\r' || *p == '\t' || *p == '\f' || *p == '\v')) ++p;
        if (p >= end) return false;
        *tok = p;
        while (p < end && !(*p == ' ' || *p == '\n' || *p == '\r' || *p == '\t' || *p == '\f' || *p == '\v')) ++p;
        *len = (size_t)(p - *tok);
        return true;
    }
};

bool parse_uint(const char* tok, size_t len, int base, uint64_t limit, uint64_t* out) {
    if (len == 0) return false;
    size_t i = 0;
    if (base == 16 && len > 2 && tok[0] == '0' && (tok[1] == 'x' || tok[1] == 'X')) i = 2;   // stream extraction accepts it
    uint64_t v = 0;
    for (; i < len; ++i) {
        const char c = tok[i];
        int d;
        if (c >= '0' && c <= '9') d = c - '0';
        else if (base == 16 && c >= 'a' && c <= 'f') d = c - 'a' + 10;
        else if (base == 16 && c >= 'A' && c <= 'F') d = c - 'A' + 10;
        else return false;
        v = v * (uint64_t)base + (uint64_t)d;
        if (v > limit) return false;
    }
    *out = v;
    return true;
}

}  // namespace

extern "C" {

int sessd_wts_load(const char* path, sessd_wts** out) {
    if (!path || !out) return SESSD_ERR_NULL;
    *out = nullptr;
    FILE* f = std::fopen(path, "rb");
    if (!f) return SESSD_ERR_IO;
    std::vector<char> buf;
    if (std::fseek(f, 0, SEEK_END) == 0) {
        const long n = std::ftell(f);
        if (n > 0) buf.resize((size_t)n);
        std::rewind(f);
    }
    size_t got = buf.empty() ? 0 : std::fread(buf.data(), 1, buf.size(), f);
    std::fclose(f);
    if (got != buf.size() || buf.empty()) return SESSD_ERR_IO;

    Tokens t{buf.data(), buf.data() + buf.size()};
    const char* tok;
    size_t len;
    uint64_t count = 0;
    if (!t.next(&tok, &len) || !parse_uint(tok, len, 10, 1u << 24, &count) || count == 0) return SESSD_ERR_IO;
    auto* w = new sessd_wts();
    w->names.reserve(count);
    w->values.reserve(count);
    for (uint64_t b = 0; b < count; ++b) {
        uint64_t size = 0;
        const char* name;
        size_t name_len;
        if (!t.next(&name, &name_len) || !t.next(&tok, &len) || !parse_uint(tok, len, 10, 0xFFFFFFFFull, &size) ||
            size * 2 > (uint64_t)(t.end - t.p) + 1) {   // every word needs at least a digit and a separator
            delete w;
            return SESSD_ERR_IO;
        }
        std::vector<float> vals((size_t)size);
        for (uint64_t i = 0; i < size; ++i) {
            uint64_t bits;
            if (!t.next(&tok, &len) || !parse_uint(tok, len, 16, 0xFFFFFFFFull, &bits)) {
                delete w;
                return SESSD_ERR_IO;
            }
            const uint32_t u = (uint32_t)bits;
            std::memcpy(&vals[(size_t)i], &u, 4);
        }
        std::string key(name, name_len);
        w->index[key] = (int)w->names.size();
        w->names.push_back(std::move(key));
        w->values.push_back(std::move(vals));
    }
    *out = w;
    return SESSD_OK;
}

void sessd_wts_destroy(sessd_wts* w) { delete w; }

int sessd_wts_count(const sessd_wts* w) { return w ? (int)w->names.size() : SESSD_ERR_NULL; }

int sessd_wts_entry(const sessd_wts* w, int i, const char** name, const float** values, int64_t* count) {
    if (!w) return SESSD_ERR_NULL;
    if (i < 0 || i >= (int)w->names.size()) return SESSD_ERR_PARAM;
    if (name) *name = w->names[(size_t)i].c_str();
    if (values) *values = w->values[(size_t)i].data();
    if (count) *count = (int64_t)w->values[(size_t)i].size();
    return SESSD_OK;
}

int sessd_wts_find(const sessd_wts* w, const char* name, const float** values, int64_t* count) {
    if (!w || !name) return SESSD_ERR_NULL;
    const auto it = w->index.find(name);
    if (it == w->index.end()) return SESSD_ERR_PARAM;
    return sessd_wts_entry(w, it->second, nullptr, values, count);
}

int sessd_wts_save(const char* path, int n, const char* const* names, const float* const* values,
                   const int64_t* counts) {
    if (!path || !names || !values || !counts) return SESSD_ERR_NULL;
    if (n < 1) return SESSD_ERR_PARAM;
    for (int b = 0; b < n; ++b) {
        if (!names[b] || (!values[b] && counts[b] > 0)) return SESSD_ERR_NULL;
        if (counts[b] < 0 || counts[b] > 0xFFFFFFFFll || names[b][0] == 0 || std::strpbrk(names[b], " \t\r\n\f\v"))
            return SESSD_ERR_PARAM;
    }
    FILE* f = std::fopen(path, "wb");
    if (!f) return SESSD_ERR_IO;
    bool ok = std::fprintf(f, "%d\n", n) > 0;
    static const char digits[] = "0123456789abcdef";
    std::vector<char> line;
    for (int b = 0; b < n && ok; ++b) {
        ok = std::fprintf(f, "%s %lld ", names[b], (long long)counts[b]) > 0;
        line.resize((size_t)counts[b] * 9 + 1);
        char* q = line.data();
        for (int64_t i = 0; i < counts[b]; ++i) {
            uint32_t u;
            std::memcpy(&u, &values[b][i], 4);
            *q++ = ' ';
            for (int s = 28; s >= 0; s -= 4) *q++ = digits[(u >> s) & 15u];
        }
        *q++ = '\n';
        ok = ok && std::fwrite(line.data(), 1, (size_t)(q - line.data()), f) == (size_t)(q - line.data());
    }
    ok = (std::fclose(f) == 0) && ok;
    return ok ? SESSD_OK : SESSD_ERR_IO;
}

int sessd_fold_batchnorm(const float* gamma, const float* beta, const float* mean, const float* var, int len,
                         float eps, float* scale, float* shift) {
    if (!gamma || !beta || !mean || !var || !scale || !shift) return SESSD_ERR_NULL;
    if (len < 1) return SESSD_ERR_PARAM;
    for (int i = 0; i < len; ++i) {
        const float root = std::sqrt(var[i] + eps);
        scale[i] = gamma[i] / root;
        shift[i] = beta[i] - mean[i] * gamma[i] / root;
    }
    return SESSD_OK;
}

int sessd_backbone_create_from_wts(const sessd_voxel_params* vp, const sessd_conv_params* layers, int nlayers,
                                   const int32_t* module_index, const sessd_wts* w, const char* prefix, float eps,
                                   const sessd_s2d_params* s2d, int dtype, sessd_backbone** out) {
    if (!vp || !layers || !module_index || !w || !prefix || !out) return SESSD_ERR_NULL;
    if (nlayers < 1 || nlayers > 64) return SESSD_ERR_PARAM;
    std::vector<const float*> weights((size_t)nlayers), scale_p((size_t)nlayers), shift_p((size_t)nlayers);
    std::vector<std::vector<float>> scale((size_t)nlayers), shift((size_t)nlayers);
    const std::string base(prefix);
    for (int l = 0; l < nlayers; ++l) {
        const sessd_conv_params& p = layers[l];
        if (p.in_channel < 1 || p.out_channel < 1) return SESSD_ERR_PARAM;
        const int64_t kvol = (int64_t)p.ksize[0] * p.ksize[1] * p.ksize[2];
        const std::string conv = base + "." + std::to_string(module_index[l]);
        const std::string bn = base + "." + std::to_string(module_index[l] + 1);
        int64_t n = 0;
        int rc = sessd_wts_find(w, (conv + ".weight").c_str(), &weights[(size_t)l], &n);
        if (rc) return rc;
        if (n != kvol * p.in_channel * p.out_channel) return SESSD_ERR_PARAM;
        const float* part[4];
        static const char* const suffix[4] = {".weight", ".bias", ".running_mean", ".running_var"};
        for (int j = 0; j < 4; ++j) {
            rc = sessd_wts_find(w, (bn + suffix[j]).c_str(), &part[j], &n);
            if (rc) return rc;
            if (n != p.out_channel) return SESSD_ERR_PARAM;
        }
        scale[(size_t)l].resize((size_t)p.out_channel);
        shift[(size_t)l].resize((size_t)p.out_channel);
        rc = sessd_fold_batchnorm(part[0], part[1], part[2], part[3], p.out_channel, eps, scale[(size_t)l].data(),
                                  shift[(size_t)l].data());
        if (rc) return rc;
        scale_p[(size_t)l] = scale[(size_t)l].data();
        shift_p[(size_t)l] = shift[(size_t)l].data();
    }
    return sessd_backbone_create(vp, layers, nlayers, weights.data(), scale_p.data(), shift_p.data(), s2d, dtype, out);
}

int sessd_points_load(const char* path, float* points, int max_points, int32_t* points_size) {
    if (!path || !points || !points_size) return SESSD_ERR_NULL;
    if (max_points < 1) return SESSD_ERR_PARAM;
    *points_size = 0;
    FILE* f = std::fopen(path, "rb");
    if (!f) return SESSD_ERR_IO;
    const size_t cap = (size_t)max_points * 16;
    const size_t got = std::fread(points, 1, cap, f);
    const bool more = got == cap && std::fgetc(f) != EOF;   // the reference gives up on a file that does not fit
    const bool bad = std::ferror(f) != 0;
    std::fclose(f);
    if (bad) return SESSD_ERR_IO;
    if (more) return SESSD_ERR_PARAM;
    std::memset(reinterpret_cast<char*>(points) + got, 0, cap - got);
    *points_size = (int32_t)(got / 16);
    return SESSD_OK;
}

}  // extern "C"
