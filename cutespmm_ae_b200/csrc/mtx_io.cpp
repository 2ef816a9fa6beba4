// MatrixMarket coordinate reader: the C-ABI replacement of MTX_READER (reference IO.cu:1-88).
//
// pattern_only mode reproduces the reference's observable result exactly: dimensions padded up to
// multiples of 16 (IO.cu:30-31), all values 1.0 (IO.cu:68,81), mirrored off-diagonal entries under a
// "symmetric" header (IO.cu:16,42,77), entries in file order inside a row.  The parser is a single
// pass over a memory buffer with strtoul/strtof instead of two getline/istringstream passes.
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "../../include/cutespmm.h"

struct cutespmm_mtx {
    uint32_t M = 0, K = 0, nnz = 0;
    std::vector<uint32_t> rowPtr, cols;
    std::vector<float> vals;
};

namespace cutespmm {
void set_last_error(const std::string &msg);  // capi.cu
}

namespace {
struct Entry {
    uint32_t r, c;
    float v;
};

int fail(int status, const std::string &path, const std::string &what)
{
    cutespmm::set_last_error("MatrixMarket file " + path + ": " + what);
    return status;
}

// Parses an unsigned decimal that must start (after blanks) before `line_end`; never reads into the next line.
bool parse_uint(const char *&p, const char *line_end, unsigned long &out)
{
    while (p < line_end && (*p == ' ' || *p == '\t')) ++p;
    if (p >= line_end || *p < '0' || *p > '9') return false;
    unsigned long v = 0;
    while (p < line_end && *p >= '0' && *p <= '9') {
        if (v > (~0ul - 9) / 10) return false;
        v = v * 10 + (unsigned long)(*p++ - '0');
    }
    out = v;
    return true;
}
}  // namespace

extern "C" {

int cutespmm_mtx_open(cutespmm_mtx_t **out, const char *path, int pattern_only)
{
    if (!out || !path) {
        cutespmm::set_last_error("cutespmm_mtx_open: null argument");
        return CUTESPMM_EINVAL;
    }
    *out = nullptr;
    FILE *f = std::fopen(path, "rb");
    if (!f) return fail(CUTESPMM_EIO, path, std::string("cannot open: ") + std::strerror(errno));
    std::fseek(f, 0, SEEK_END);
    const long size = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    if (size <= 0) { std::fclose(f); return fail(CUTESPMM_EIO, path, "empty or unreadable"); }
    std::string buf((size_t)size, '\0');
    const size_t got = std::fread(&buf[0], 1, (size_t)size, f);
    std::fclose(f);
    if (got != (size_t)size) return fail(CUTESPMM_EIO, path, "short read");

    const char *p = buf.c_str(), *end = p + buf.size();
    auto next_line = [&](const char *q) { while (q < end && *q != '\n') ++q; return q < end ? q + 1 : end; };
    // header line: the reference only looks for the word "symmetric" (IO.cu:15-16)
    const char *l1 = next_line(p);
    const bool symmetric = std::string(p, l1).find("symmetric") != std::string::npos;
    p = l1;
    size_t line_no = 2;
    while (p < end && *p == '%') { p = next_line(p); ++line_no; }
    if (p >= end) return fail(CUTESPMM_EIO, path, "no size line");
    unsigned long m0 = 0, k0 = 0;
    {
        const char *size_end = next_line(p), *q = p;
        if (!parse_uint(q, size_end, m0) || !parse_uint(q, size_end, k0) || m0 == 0 || k0 == 0 || m0 >= (1ul << 32) - 16 ||
            k0 >= (1ul << 32) - 16)
            return fail(CUTESPMM_EIO, path, "bad size line (line " + std::to_string(line_no) + ")");
        p = size_end;
    }

    cutespmm_mtx *m = new (std::nothrow) cutespmm_mtx();
    if (!m) return fail(CUTESPMM_ENOMEM, path, "host allocation failed");
    m->M = (uint32_t)((m0 - 1) / 16 + 1) * 16;
    m->K = (uint32_t)((k0 - 1) / 16 + 1) * 16;
    std::vector<Entry> ents;
    while (p < end) {
        const char *line_end = next_line(p);
        ++line_no;
        while (p < line_end && (*p == ' ' || *p == '\t' || *p == '\r')) ++p;
        if (p >= line_end || *p == '\n' || *p == '%') { p = line_end; continue; }
        unsigned long r = 0, c = 0;
        const char *q = p;
        if (!parse_uint(q, line_end, r) || !parse_uint(q, line_end, c)) {
            delete m;
            return fail(CUTESPMM_EIO, path, "line " + std::to_string(line_no) + ": expected a row and a column index");
        }
        // a mirrored entry (c, r) must lie inside the declared matrix too
        if (r == 0 || c == 0 || r > m0 || c > k0 || (symmetric && (c > m0 || r > k0))) {
            delete m;
            return fail(CUTESPMM_EIO, path, "line " + std::to_string(line_no) + ": index outside the " + std::to_string(m0) + " x " +
                                                std::to_string(k0) + " matrix" + (symmetric ? " (or its mirror image is)" : ""));
        }
        float v = 1.0f;
        if (!pattern_only) {
            const char *t = q;
            while (t < line_end && (*t == ' ' || *t == '\t')) ++t;
            if (t < line_end && *t != '\n' && *t != '\r') v = std::strtof(t, nullptr);
        }
        ents.push_back(Entry{(uint32_t)(r - 1), (uint32_t)(c - 1), v});
        p = line_end;
    }
    // counting sort by row keeping file order; a mirrored entry follows its original (IO.cu:71-84)
    m->rowPtr.assign((size_t)m->M + 1, 0);
    for (const Entry &e : ents) {
        ++m->rowPtr[e.r + 1];
        if (symmetric && e.r != e.c) ++m->rowPtr[e.c + 1];
    }
    for (size_t i = 0; i < m->M; ++i) m->rowPtr[i + 1] += m->rowPtr[i];
    m->nnz = m->rowPtr[m->M];
    m->cols.resize(m->nnz);
    m->vals.resize(m->nnz);
    std::vector<uint32_t> cursor(m->rowPtr.begin(), m->rowPtr.end() - 1);
    for (const Entry &e : ents) {
        m->cols[cursor[e.r]] = e.c;
        m->vals[cursor[e.r]++] = e.v;
        if (symmetric && e.r != e.c) {
            m->cols[cursor[e.c]] = e.r;
            m->vals[cursor[e.c]++] = e.v;
        }
    }
    *out = m;
    return CUTESPMM_OK;
}

int cutespmm_mtx_dims(const cutespmm_mtx_t *m, uint32_t *M, uint32_t *K, uint32_t *nnz)
{
    if (!m) return CUTESPMM_EINVAL;
    if (M) *M = m->M;
    if (K) *K = m->K;
    if (nnz) *nnz = m->nnz;
    return CUTESPMM_OK;
}

int cutespmm_mtx_arrays(const cutespmm_mtx_t *m, const uint32_t **rowPtr, const uint32_t **cols, const float **vals)
{
    if (!m) return CUTESPMM_EINVAL;
    if (rowPtr) *rowPtr = m->rowPtr.data();
    if (cols) *cols = m->cols.data();
    if (vals) *vals = m->vals.data();
    return CUTESPMM_OK;
}

int cutespmm_mtx_close(cutespmm_mtx_t *m)
{
    delete m;
    return CUTESPMM_OK;
}

}  // extern "C"
