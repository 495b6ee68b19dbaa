// .smtx text reader/writer and CSR validation (host side, no CUDA).
//
// File format (dlmc/README:5 in the reference data set): first line "M, K, nnz", second line
// M+1 row offsets, third line nnz column indices, all decimal integers.  The reference parses it
// with fscanf("%d,%d,%d") followed by one fscanf("%d") per number
// (SPMM/spmm-esimd-fromfile.cpp:105-137); any whitespace separates numbers.  This reader accepts
// the same texts and produces the same integers, reading the file in one piece.
#include <errno.h>
#include <limits.h>
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

}  // namespace

extern "C" int dlspm_read_smtx_host(const char *path, int *M, int *K, int *nnz, int **row_offsets,
                                    int **column_indices)
{
    if (!path || !M || !K || !nnz || !row_offsets || !column_indices) return DLSPM_ERR_INVALID_ARGUMENT;
    *row_offsets = nullptr;
    *column_indices = nullptr;
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
    free(text);
    if (rc != DLSPM_OK) {
        free(ro);
        free(ci);
        return rc;
    }
    *M = m;
    *K = k;
    *nnz = z;
    *row_offsets = ro;
    *column_indices = ci;
    return DLSPM_OK;
}

extern "C" int dlspm_write_smtx_host(const char *path, int M, int K, int nnz, const int *row_offsets,
                                     const int *column_indices)
{
    if (!path || M < 0 || K < 0 || nnz < 0 || !row_offsets || (nnz > 0 && !column_indices))
        return DLSPM_ERR_INVALID_ARGUMENT;
    FILE *fp = fopen(path, "wb");
    if (!fp) return DLSPM_ERR_IO;
    fprintf(fp, "%d, %d, %d\n", M, K, nnz);
    for (int i = 0; i <= M; i++) fprintf(fp, i == M ? "%d\n" : "%d ", row_offsets[i]);
    for (int i = 0; i < nnz; i++) fprintf(fp, i == nnz - 1 ? "%d\n" : "%d ", column_indices[i]);
    if (nnz == 0) fprintf(fp, "\n");
    const bool bad = ferror(fp) != 0;
    if (fclose(fp) != 0 || bad) return DLSPM_ERR_IO;
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
