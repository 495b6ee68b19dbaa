// .smtx text reader/writer and CSR validation (host side, no CUDA).
//
// File format (dlmc/README:5 in the reference data set): first line "M, K, nnz", second line
// M+1 row offsets, third line nnz column indices, all decimal integers.  The reference parses it
// with fscanf("%d,%d,%d") followed by one fscanf("%d") per number
// (SPMM/spmm-esimd-fromfile.cpp:105-137); any whitespace separates numbers.  This reader accepts
// the same texts and produces the same integers, reading the file in one piece.
//
// Two additions the reference does not have (it invents values with rand() and re-parses the text
// on every run): an optional fourth block of nnz decimal floats after the indices, which the
// plain readers (this one and the reference's) skip, and a binary cache of a parsed matrix.
#include <errno.h>
#include <limits.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>

#include "../../include/dlspm.h"

namespace {

inline bool is_space(char c) { return c == ' ' || c == '\n' || c == '\t' || c == '\r' || c == '\f' || c == '\v'; }

// Parses one decimal int the way scanf's %d does: optional whitespace, optional sign, digits.
bool parse_int(const char *&p, const char *end, int *out)
{
    while (p < end && is_space(*p)) p++;
    if (p >= end) return false;
    bool neg = false;
    if (*p == '-' || *p == '+') {
        neg = (*p == '-');
        p++;
    }
    if (p >= end || *p < '0' || *p > '9') return false;
    long long v = 0;
    while (p < end && *p >= '0' && *p <= '9') {
        v = v * 10 + (*p - '0');
        if (v > (long long)INT_MAX + 1) return false;
        p++;
    }
    if (neg) v = -v;
    if (v > INT_MAX || v < INT_MIN) return false;
    *out = (int)v;
    return true;
}

// A literal ',' directly after the previous number, as in the scanf format "%d,%d,%d".
bool expect_comma(const char *&p, const char *end)
{
    if (p < end && *p == ',') {
        p++;
        return true;
    }
    return false;
}

// Parses one float the way scanf's %f does (strtof on a NUL-terminated buffer).
bool parse_float(const char *&p, const char *end, float *out)
{
    while (p < end && is_space(*p)) p++;
    if (p >= end) return false;
    char *stop = nullptr;
    errno = 0;
    const float v = strtof(p, &stop);
    if (stop == p) return false;
    p = stop;
    *out = v;
    return true;
}

// Reads the text; `values` may be NULL (plain reader).  With `values`, a fourth block of nnz
// decimal floats after the column indices is parsed if the file has one; *values stays NULL if
// it has none.
int read_smtx(const char *path, int *M, int *K, int *nnz, int **row_offsets, int **column_indices,
              float **values)
{
    if (!path || !M || !K || !nnz || !row_offsets || !column_indices) return DLSPM_ERR_INVALID_ARGUMENT;
    *row_offsets = nullptr;
    *column_indices = nullptr;
    if (values) *values = nullptr;
    FILE *fp = fopen(path, "rb");
    if (!fp) return DLSPM_ERR_IO;
    if (fseek(fp, 0, SEEK_END) != 0) {
        fclose(fp);
        return DLSPM_ERR_IO;
    }
    long size = ftell(fp);
    if (size < 0 || fseek(fp, 0, SEEK_SET) != 0) {
        fclose(fp);
        return DLSPM_ERR_IO;
    }
    char *text = (char *)malloc((size_t)size + 1);
    if (!text) {
        fclose(fp);
        return DLSPM_ERR_NOMEM;
    }
    size_t got = fread(text, 1, (size_t)size, fp);
    fclose(fp);
    text[got] = 0;
    const char *p = text, *end = text + got;

    int m = 0, k = 0, z = 0;
    int rc = DLSPM_OK;
    int *ro = nullptr, *ci = nullptr;
    float *va = nullptr;
    if (!parse_int(p, end, &m) || !expect_comma(p, end) || !parse_int(p, end, &k) ||
        !expect_comma(p, end) || !parse_int(p, end, &z) || m < 0 || k < 0 || z < 0) {
        rc = DLSPM_ERR_FORMAT;
    }
    if (rc == DLSPM_OK) {
        ro = (int *)malloc(((size_t)m + 1) * sizeof(int));
        ci = (int *)malloc(((size_t)z > 0 ? (size_t)z : 1) * sizeof(int));
        if (!ro || !ci) rc = DLSPM_ERR_NOMEM;
    }
    for (int i = 0; rc == DLSPM_OK && i < m + 1; i++) {
        if (!parse_int(p, end, &ro[i])) rc = DLSPM_ERR_FORMAT;
    }
    for (int i = 0; rc == DLSPM_OK && i < z; i++) {
        if (!parse_int(p, end, &ci[i])) rc = DLSPM_ERR_FORMAT;
    }
    if (rc == DLSPM_OK && values) {
        while (p < end && is_space(*p)) p++;
        if (p < end) {  // something follows the indices: it must be exactly nnz floats
            va = (float *)malloc(((size_t)z > 0 ? (size_t)z : 1) * sizeof(float));
            if (!va) rc = DLSPM_ERR_NOMEM;
            for (int i = 0; rc == DLSPM_OK && i < z; i++) {
                if (!parse_float(p, end, &va[i])) rc = DLSPM_ERR_FORMAT;
            }
        }
    }
    free(text);
    if (rc != DLSPM_OK) {
        free(ro);
        free(ci);
        free(va);
        return rc;
    }
    *M = m;
    *K = k;
    *nnz = z;
    *row_offsets = ro;
    *column_indices = ci;
    if (values) *values = va;
    return DLSPM_OK;
}

int write_smtx(const char *path, int M, int K, int nnz, const int *row_offsets, const int *column_indices,
               const float *values)
{
    if (!path || M < 0 || K < 0 || nnz < 0 || !row_offsets || (nnz > 0 && !column_indices))
        return DLSPM_ERR_INVALID_ARGUMENT;
    FILE *fp = fopen(path, "wb");
    if (!fp) return DLSPM_ERR_IO;
    fprintf(fp, "%d, %d, %d\n", M, K, nnz);
    for (int i = 0; i <= M; i++) fprintf(fp, i == M ? "%d\n" : "%d ", row_offsets[i]);
    for (int i = 0; i < nnz; i++) fprintf(fp, i == nnz - 1 ? "%d\n" : "%d ", column_indices[i]);
    if (nnz == 0) fprintf(fp, "\n");
    // nine significant digits give back every fp32 value exactly
    if (values)
        for (int i = 0; i < nnz; i++) fprintf(fp, i == nnz - 1 ? "%.9g\n" : "%.9g ", (double)values[i]);
    const bool bad = ferror(fp) != 0;
    if (fclose(fp) != 0 || bad) return DLSPM_ERR_IO;
    return DLSPM_OK;
}

// ---- binary CSR cache -------------------------------------------------------------------------
// Little-endian file: a 48-byte header, then row_offsets, column_indices and (optionally) values,
// each block padded with zeros to a multiple of 8 bytes.  The checksum covers the three blocks.
struct CacheHeader {
    char magic[8];       // "DLSPMCSR"
    uint32_t version;    // 1
    uint32_t flags;      // bit 0: the file carries values
    int32_t M, K, nnz;
    uint32_t reserved;
    uint64_t checksum;
    uint64_t payload_bytes;
};
static_assert(sizeof(CacheHeader) == 48, "header layout");
const char kCacheMagic[8] = {'D', 'L', 'S', 'P', 'M', 'C', 'S', 'R'};

inline size_t pad8(size_t n) { return (n + 7) & ~(size_t)7; }

// 64-bit multiply-xorshift over 8-byte words (position dependent, cheap, not cryptographic)
uint64_t fold_words(uint64_t h, const void *data, size_t bytes)
{
    const unsigned char *p = (const unsigned char *)data;
    for (size_t i = 0; i < bytes; i += 8) {
        uint64_t w = 0;
        memcpy(&w, p + i, bytes - i < 8 ? bytes - i : 8);
        h = (h ^ w) * 0x9E3779B97F4A7C15ull;
        h ^= h >> 29;
    }
    return h;
}

bool write_padded(FILE *fp, const void *data, size_t bytes)
{
    static const char zeros[8] = {0};
    if (bytes && fwrite(data, 1, bytes, fp) != bytes) return false;
    const size_t tail = pad8(bytes) - bytes;
    return tail == 0 || fwrite(zeros, 1, tail, fp) == tail;
}

bool read_padded(FILE *fp, void *data, size_t bytes)
{
    char skip[8];
    if (bytes && fread(data, 1, bytes, fp) != bytes) return false;
    const size_t tail = pad8(bytes) - bytes;
    return tail == 0 || fread(skip, 1, tail, fp) == tail;
}

}  // namespace

extern "C" int dlspm_read_smtx_host(const char *path, int *M, int *K, int *nnz, int **row_offsets,
                                    int **column_indices)
{
    return read_smtx(path, M, K, nnz, row_offsets, column_indices, nullptr);
}

extern "C" int dlspm_read_smtx_values_host(const char *path, int *M, int *K, int *nnz, int **row_offsets,
                                           int **column_indices, float **values)
{
    if (!values) return DLSPM_ERR_INVALID_ARGUMENT;
    return read_smtx(path, M, K, nnz, row_offsets, column_indices, values);
}

extern "C" int dlspm_write_smtx_host(const char *path, int M, int K, int nnz, const int *row_offsets,
                                     const int *column_indices)
{
    return write_smtx(path, M, K, nnz, row_offsets, column_indices, nullptr);
}

extern "C" int dlspm_write_smtx_values_host(const char *path, int M, int K, int nnz, const int *row_offsets,
                                            const int *column_indices, const float *values)
{
    if (nnz > 0 && !values) return DLSPM_ERR_INVALID_ARGUMENT;
    return write_smtx(path, M, K, nnz, row_offsets, column_indices, values);
}

extern "C" int dlspm_write_csr_cache_host(const char *path, int M, int K, int nnz, const int *row_offsets,
                                          const int *column_indices, const float *values)
{
    if (!path || M < 0 || K < 0 || nnz < 0 || !row_offsets || (nnz > 0 && !column_indices))
        return DLSPM_ERR_INVALID_ARGUMENT;
    const size_t ro_bytes = 4 * ((size_t)M + 1), ci_bytes = 4 * (size_t)nnz, va_bytes = values ? 4 * (size_t)nnz : 0;
    CacheHeader h;
    memset(&h, 0, sizeof h);
    memcpy(h.magic, kCacheMagic, 8);
    h.version = 1;
    h.flags = values ? 1u : 0u;
    h.M = M;
    h.K = K;
    h.nnz = nnz;
    h.payload_bytes = pad8(ro_bytes) + pad8(ci_bytes) + pad8(va_bytes);
    uint64_t sum = fold_words(0x243F6A8885A308D3ull, row_offsets, ro_bytes);
    sum = fold_words(sum, column_indices, ci_bytes);
    if (values) sum = fold_words(sum, values, va_bytes);
    h.checksum = sum;
    FILE *fp = fopen(path, "wb");
    if (!fp) return DLSPM_ERR_IO;
    bool ok = fwrite(&h, 1, sizeof h, fp) == sizeof h && write_padded(fp, row_offsets, ro_bytes) &&
              write_padded(fp, column_indices, ci_bytes) && write_padded(fp, values, va_bytes);
    ok = ok && ferror(fp) == 0;
    if (fclose(fp) != 0 || !ok) return DLSPM_ERR_IO;
    return DLSPM_OK;
}

extern "C" int dlspm_read_csr_cache_host(const char *path, int *M, int *K, int *nnz, int **row_offsets,
                                         int **column_indices, float **values)
{
    if (!path || !M || !K || !nnz || !row_offsets || !column_indices || !values) return DLSPM_ERR_INVALID_ARGUMENT;
    *row_offsets = nullptr;
    *column_indices = nullptr;
    *values = nullptr;
    FILE *fp = fopen(path, "rb");
    if (!fp) return DLSPM_ERR_IO;
    CacheHeader h;
    if (fread(&h, 1, sizeof h, fp) != sizeof h || memcmp(h.magic, kCacheMagic, 8) != 0 || h.version != 1 ||
        (h.flags & ~1u) || h.M < 0 || h.K < 0 || h.nnz < 0) {
        fclose(fp);
        return DLSPM_ERR_FORMAT;
    }
    const bool has_values = (h.flags & 1u) != 0;
    const size_t ro_bytes = 4 * ((size_t)h.M + 1), ci_bytes = 4 * (size_t)h.nnz, va_bytes = has_values ? 4 * (size_t)h.nnz : 0;
    if (h.payload_bytes != pad8(ro_bytes) + pad8(ci_bytes) + pad8(va_bytes)) {
        fclose(fp);
        return DLSPM_ERR_FORMAT;
    }
    // the sizes in the header must agree with the file before anything is allocated from them
    if (fseek(fp, 0, SEEK_END) != 0 || ftell(fp) < 0 || (uint64_t)ftell(fp) != sizeof h + h.payload_bytes ||
        fseek(fp, (long)sizeof h, SEEK_SET) != 0) {
        fclose(fp);
        return DLSPM_ERR_FORMAT;
    }
    int *ro = (int *)malloc(ro_bytes);
    int *ci = (int *)malloc(ci_bytes ? ci_bytes : 4);
    float *va = has_values ? (float *)malloc(va_bytes ? va_bytes : 4) : nullptr;
    int rc = DLSPM_OK;
    if (!ro || !ci || (has_values && !va)) rc = DLSPM_ERR_NOMEM;
    if (rc == DLSPM_OK && !(read_padded(fp, ro, ro_bytes) && read_padded(fp, ci, ci_bytes) && read_padded(fp, va, va_bytes)))
        rc = DLSPM_ERR_FORMAT;
    fclose(fp);
    if (rc == DLSPM_OK) {
        uint64_t sum = fold_words(0x243F6A8885A308D3ull, ro, ro_bytes);
        sum = fold_words(sum, ci, ci_bytes);
        if (has_values) sum = fold_words(sum, va, va_bytes);
        if (sum != h.checksum) rc = DLSPM_ERR_FORMAT;
    }
    if (rc != DLSPM_OK) {
        free(ro);
        free(ci);
        free(va);
        return rc;
    }
    *M = h.M;
    *K = h.K;
    *nnz = h.nnz;
    *row_offsets = ro;
    *column_indices = ci;
    *values = va;
    return DLSPM_OK;
}

// The checks of the reference's SanityCheck in its order, with its exception texts
// (SPMM/spmm-esimd-fromfile.cpp:36-61), then the two checks it leaves out.
extern "C" int dlspm_sanity_check_csr_host(int M, int K, int N, int nnz, const int *row_offsets,
                                           const int *column_indices, char *why, size_t why_len)
{
    const char *msg = nullptr;
    if (M < 0 || K < 0 || N < 0 || nnz < 0 || !row_offsets || (nnz > 0 && !column_indices)) {
        if (why && why_len) snprintf(why, why_len, "invalid argument");
        return DLSPM_ERR_INVALID_ARGUMENT;
    }
    if ((long long)nnz > (long long)M * (long long)K) msg = "nnz is larger than matrix.";
    else if (row_offsets[M] != nnz) msg = "a_row_offsets[MSZ] != nnz.";
    for (int i = 0; i < M && !msg; i++) {
        if (row_offsets[i + 1] < row_offsets[i]) msg = "a_row_offsets[i+1] < a_row_offsets[i]";
        else if (row_offsets[i + 1] - row_offsets[i] > K) msg = "a_row_offsets[i + 1] - a_row_offsets[i] > KSZ";
    }
    for (int i = 0; i < nnz && !msg; i++) {
        if (column_indices[i] >= K) msg = "a_column_indices[i] >= KSZ";
    }
    if (!msg && row_offsets[0] != 0) msg = "a_row_offsets[0] != 0";
    for (int i = 0; i < nnz && !msg; i++) {
        if (column_indices[i] < 0) msg = "a_column_indices[i] < 0";
    }
    if (why && why_len) snprintf(why, why_len, "%s", msg ? msg : "");
    return msg ? DLSPM_ERR_CSR : DLSPM_OK;
}
