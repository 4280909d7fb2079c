// Host-side reader / writer of the three-line ".smtx" text format that carries matrices between the
// two stages: "rows, cols, nnz" / row pointers / column ids, single spaces, no newline after the last
// column id.  Written by the reference's CVSE_out (RowMerge/sparse_matrix_format.py:152-175) and by
// the DLMC dataset; parsed by the reference's driver (SSpMM/sspmm_test.cpp:28-64) and reader
// (RowMerge/sparse_matrix_format.py:8-25).  Plain C++ on host memory; no CUDA call.
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/sspmm_b200.h"
#include "launch.h"

namespace sspmm_b200 {
namespace {

bool read_file(const char* path, std::string& out) {
    FILE* f = std::fopen(path, "rb");
    if (!f) return false;
    std::fseek(f, 0, SEEK_END);
    const long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    out.resize(n > 0 ? (size_t)n : 0);
    const size_t got = n > 0 ? std::fread(&out[0], 1, (size_t)n, f) : 0;
    std::fclose(f);
    return got == out.size();
}

// Parses non-negative decimal integers separated by spaces from [p, end) up to a newline; returns the
// position after the newline (or end).  Stores at most `cap` values, counts all of them.
const char* parse_line(const char* p, const char* end, int* dst, long long cap, long long& count, bool& ok) {
    count = 0;
    while (p < end && *p != '\n') {
        while (p < end && (*p == ' ' || *p == '\r' || *p == '\t')) ++p;
        if (p >= end || *p == '\n') break;
        long long v = 0;
        bool neg = false, any = false;
        if (*p == '-') { neg = true; ++p; }
        while (p < end && *p >= '0' && *p <= '9') { v = v * 10 + (*p - '0'); ++p; any = true; if (v > 0x7fffffffLL) ok = false; }
        if (!any) { ok = false; return end; }
        if (dst && count < cap) dst[count] = (int)(neg ? -v : v);
        ++count;
    }
    return p < end ? p + 1 : end;
}

bool parse_header(const char*& p, const char* end, int hdr[3]) {
    // "rows, cols, nnz\n": commas and optional blanks
    for (int k = 0; k < 3; ++k) {
        while (p < end && (*p == ' ' || *p == ',')) ++p;
        long long v = 0;
        bool any = false;
        while (p < end && *p >= '0' && *p <= '9') { v = v * 10 + (*p - '0'); ++p; any = true; }
        if (!any || v > 0x7fffffffLL) return false;
        hdr[k] = (int)v;
    }
    while (p < end && *p != '\n') ++p;
    if (p < end) ++p;
    return true;
}

int io_error(const char* what, const char* path) {
    set_error("%s '%s': %s", what, path, errno ? std::strerror(errno) : "malformed file");
    return 1;
}

}  // namespace
}  // namespace sspmm_b200

using namespace sspmm_b200;

extern "C" int smtx_read_header(const char* path, int* rows, int* cols, int* nnz, int64_t* n_row_ptr, int64_t* n_col_idx) {
    std::string buf;
    errno = 0;
    if (!path || !read_file(path, buf)) return io_error("cannot read", path ? path : "(null)");
    const char* p = buf.data();
    const char* end = p + buf.size();
    int hdr[3];
    errno = 0;
    if (!parse_header(p, end, hdr)) return io_error("bad header in", path);
    bool ok = true;
    long long n1 = 0, n2 = 0;
    p = parse_line(p, end, nullptr, 0, n1, ok);
    p = parse_line(p, end, nullptr, 0, n2, ok);
    if (!ok) return io_error("bad number in", path);
    if (rows) *rows = hdr[0];
    if (cols) *cols = hdr[1];
    if (nnz) *nnz = hdr[2];
    if (n_row_ptr) *n_row_ptr = n1;
    if (n_col_idx) *n_col_idx = n2;
    return 0;
}

extern "C" int smtx_read(const char* path, int* row_ptr, int64_t n_row_ptr, int* col_idx, int64_t n_col_idx) {
    std::string buf;
    errno = 0;
    if (!path || !read_file(path, buf)) return io_error("cannot read", path ? path : "(null)");
    const char* p = buf.data();
    const char* end = p + buf.size();
    int hdr[3];
    errno = 0;
    if (!parse_header(p, end, hdr)) return io_error("bad header in", path);
    bool ok = true;
    long long n1 = 0, n2 = 0;
    p = parse_line(p, end, row_ptr, n_row_ptr, n1, ok);
    p = parse_line(p, end, col_idx, n_col_idx, n2, ok);
    if (!ok || n1 != n_row_ptr || n2 != n_col_idx) {
        set_error("'%s' holds %lld row pointers and %lld column ids, caller expected %lld and %lld", path, n1, n2,
                  (long long)n_row_ptr, (long long)n_col_idx);
        return 1;
    }
    return 0;
}

extern "C" int smtx_write(const char* path, int rows, int cols, int nnz, const int* row_ptr, int64_t n_row_ptr,
                          const int* col_idx, int64_t n_col_idx) {
    errno = 0;
    FILE* f = path ? std::fopen(path, "wb") : nullptr;
    if (!f) return io_error("cannot write", path ? path : "(null)");
    std::vector<char> out;
    out.reserve((size_t)(n_row_ptr + n_col_idx) * 7 + 64);
    char tmp[64];
    int n = std::snprintf(tmp, sizeof tmp, "%d, %d, %d\n", rows, cols, nnz);
    out.insert(out.end(), tmp, tmp + n);
    auto put_line = [&](const int* v, int64_t cnt) {
        for (int64_t i = 0; i < cnt; ++i) {
            char b[16];
            int len = 0;
            long long x = v[i];
            const bool neg = x < 0;
            if (neg) x = -x;
            do { b[len++] = (char)('0' + x % 10); x /= 10; } while (x);
            if (neg) b[len++] = '-';
            while (len) out.push_back(b[--len]);
            if (i + 1 < cnt) out.push_back(' ');
        }
    };
    put_line(row_ptr, n_row_ptr);
    out.push_back('\n');
    put_line(col_idx, n_col_idx);
    const bool ok = std::fwrite(out.data(), 1, out.size(), f) == out.size();
    if (std::fclose(f) != 0 || !ok) return io_error("cannot write", path);
    return 0;
}
