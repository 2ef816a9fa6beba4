// Host-side containers with the surface of the reference's loaders, implemented from scratch:
//   SparseCoo<T>   (reference inc/SparseCoo.hpp:42-390)  MatrixMarket file -> sorted coordinate list
//   CSR_Matrix<T>  (reference inc/CSR.hpp:42-187, 300-340)  coordinate list or dense matrix -> CSR
//   SMA            (reference inc/SMA.hpp:1-94)  simple moving average over a fixed window
// plus cutespmm_plan_from_csr(), which hands a CSR_Matrix<float> to libcutespmm.
//
// Same public field and method names for the parts a driver uses (dimY/dimX/nnz/data_vector,
// rows/cols/values after prepare_for_cusparse(), Insert_Next, setDim, save_mtx; nrows/ncols/nnz/
// values/cols/rowPtr, ToDense).  Behaviour kept: values are read from the file (1.0 when a line has
// none), a "symmetric" header mirrors off-diagonal entries and counts them in nnz, indices become
// 0-based, entries end up ordered by (row, column).  Behaviour dropped: progress chatter on stdout,
// and the reference's comparator that answers "less" for equal elements (inc/SparseCoo.hpp:35-40) --
// ordering here is a strict weak order, stable for equal (row, column).
// The BCOO / BCSR / Blocked-ELL conversions of the reference feed library baselines and are not part
// of this path.
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "cutespmm.h"

template <class T> struct data_point {
    int row;
    int col;
    T val;
    data_point(int x, int y, T v) : row(x), col(y), val(v) {}
};

template <class DType> struct SparseCoo {
    std::vector<data_point<DType>> data_vector;
    int dimY = 0;  // rows
    int dimX = 0;  // columns
    int nnz = 0;
    int *rows = nullptr;
    int *cols = nullptr;
    DType *values = nullptr;

    SparseCoo() = default;
    SparseCoo(int dY, int dX, int nnz_) : dimY(dY), dimX(dX), nnz(nnz_) {}
    // inc/SparseCoo.hpp:91-157
    explicit SparseCoo(const std::string &FilePath)
    {
        std::ifstream infile(FilePath);
        if (!infile) throw std::runtime_error("SparseCoo: cannot open " + FilePath);
        std::string line;
        std::getline(infile, line);
        const bool symmetric = line.find("symmetric") != std::string::npos;
        while (std::getline(infile, line))
            if (line.empty() || line[0] != '%') break;
        {
            std::istringstream iss(line);
            if (!(iss >> dimY >> dimX >> nnz)) throw std::runtime_error("SparseCoo: bad size line in " + FilePath);
        }
        data_vector.reserve((size_t)nnz * (symmetric ? 2 : 1));
        while (std::getline(infile, line)) {
            std::istringstream iss(line);
            unsigned int x, y;
            double vt = 1.0;
            if (!(iss >> x >> y)) continue;
            iss >> vt;  // stays 1.0 when the line carries no value
            const DType v = (DType)vt;
            data_vector.emplace_back((int)x - 1, (int)y - 1, v);
            if (symmetric && x != y) {
                data_vector.emplace_back((int)y - 1, (int)x - 1, v);
                nnz++;
            }
        }
        sort_entries();
    }
    ~SparseCoo()
    {
        delete[] rows;
        delete[] cols;
        delete[] values;
    }
    SparseCoo(const SparseCoo &) = delete;
    SparseCoo &operator=(const SparseCoo &) = delete;

    int getX() const { return dimX; }
    int getY() const { return dimY; }
    void setDim(int dimY_, int dimX_)  // inc/SparseCoo.hpp:238-243: also forgets the entry count
    {
        dimY = dimY_;
        dimX = dimX_;
        nnz = 0;
    }
    void Insert_Next(int row, int col, DType val)
    {
        data_vector.emplace_back(row, col, val);
        nnz++;
    }
    void sort_entries()
    {
        std::stable_sort(data_vector.begin(), data_vector.end(), [](const data_point<DType> &a, const data_point<DType> &b) {
            return a.row != b.row ? a.row < b.row : a.col < b.col;
        });
    }
    // inc/SparseCoo.hpp:250-262: flat arrays for a library call
    void prepare_for_cusparse()
    {
        delete[] rows; delete[] cols; delete[] values;
        rows = new int[data_vector.size()];
        cols = new int[data_vector.size()];
        values = new DType[data_vector.size()];
        for (size_t i = 0; i < data_vector.size(); ++i) {
            rows[i] = data_vector[i].row;
            cols[i] = data_vector[i].col;
            values[i] = data_vector[i].val;
        }
    }
    // inc/SparseCoo.hpp:263-286: general coordinate file, 1-based
    void save_mtx(const std::string &out_filePath) const
    {
        std::ofstream out(out_filePath);
        if (!out) throw std::runtime_error("SparseCoo: cannot write " + out_filePath);
        out << "%%MatrixMarket matrix coordinate real general\n" << dimY << " " << dimX << " " << data_vector.size() << "\n";
        for (const auto &p : data_vector) out << p.row + 1 << " " << p.col + 1 << " " << p.val << "\n";
    }
};

template <class DType> struct CSR_Matrix {
    int nrows = 0;
    int ncols = 0;
    int nnz = 0;
    DType *values = nullptr;
    int *cols = nullptr;
    int *rowPtr = nullptr;

    CSR_Matrix() = default;
    explicit CSR_Matrix(SparseCoo<DType> &S) { coo2CSR(S); }
    CSR_Matrix(const DType *S, int m, int n) { DenseToCSR(S, m, n); }
    ~CSR_Matrix() { release(); }
    CSR_Matrix(const CSR_Matrix &) = delete;
    CSR_Matrix &operator=(const CSR_Matrix &) = delete;

    // inc/CSR.hpp:162-187: orders the coordinate list by (row, column), then counts rows
    void coo2CSR(SparseCoo<DType> &S)
    {
        release();
        S.sort_entries();
        nrows = S.dimY;
        ncols = S.dimX;
        nnz = (int)S.data_vector.size();
        rowPtr = new int[nrows + 1]();
        cols = new int[nnz > 0 ? nnz : 1];
        values = new DType[nnz > 0 ? nnz : 1];
        for (int i = 0; i < nnz; ++i) {
            const auto &p = S.data_vector[i];
            if (p.row < 0 || p.row >= nrows || p.col < 0 || p.col >= ncols) throw std::out_of_range("CSR_Matrix: entry outside the matrix");
            values[i] = p.val;
            cols[i] = p.col;
            rowPtr[p.row + 1]++;
        }
        for (int i = 0; i < nrows; ++i) rowPtr[i + 1] += rowPtr[i];
    }
    // inc/CSR.hpp DenseToCSR: keeps the entries that are not exactly zero
    void DenseToCSR(const DType *S, int m, int n)
    {
        release();
        nrows = m;
        ncols = n;
        nnz = 0;
        for (size_t i = 0; i < (size_t)m * n; ++i) nnz += S[i] != (DType)0;
        rowPtr = new int[m + 1]();
        cols = new int[nnz > 0 ? nnz : 1];
        values = new DType[nnz > 0 ? nnz : 1];
        int k = 0;
        for (int r = 0; r < m; ++r) {
            for (int c = 0; c < n; ++c)
                if (S[(size_t)r * n + c] != (DType)0) {
                    cols[k] = c;
                    values[k++] = S[(size_t)r * n + c];
                }
            rowPtr[r + 1] = k;
        }
    }
    // row-major dense copy (duplicates add up)
    std::vector<DType> ToDense() const
    {
        std::vector<DType> d((size_t)nrows * ncols, (DType)0);
        for (int r = 0; r < nrows; ++r)
            for (int j = rowPtr[r]; j < rowPtr[r + 1]; ++j) d[(size_t)r * ncols + cols[j]] += values[j];
        return d;
    }

private:
    void release()
    {
        delete[] values; delete[] cols; delete[] rowPtr;
        values = nullptr; cols = nullptr; rowPtr = nullptr;
    }
};

// inc/SMA.hpp: moving average of the last `period` samples
class SMA {
public:
    explicit SMA(unsigned int period) : period_(period ? period : 1), window_(period_, 0.0) {}
    void add(double v)
    {
        if (count_ == period_) total_ -= window_[head_];
        else ++count_;
        window_[head_] = v;
        total_ += v;
        head_ = (head_ + 1) % period_;
    }
    double avg() const { return count_ ? total_ / count_ : 0.0; }
    void reset()
    {
        std::fill(window_.begin(), window_.end(), 0.0);
        head_ = count_ = 0;
        total_ = 0.0;
    }

private:
    unsigned int period_, head_ = 0, count_ = 0;
    std::vector<double> window_;
    double total_ = 0.0;
};

// CSR_Matrix<float> -> device plan (what HRPB's constructor does for MTX_READER's arrays, data.cu:80).
inline int cutespmm_plan_from_csr(cutespmm_plan_t **plan, const CSR_Matrix<float> &A, const cutespmm_options_t *opts = nullptr,
                                  bool host_only = false)
{
    std::vector<uint64_t> rp((size_t)A.nrows + 1);
    for (int i = 0; i <= A.nrows; ++i) rp[i] = (uint64_t)A.rowPtr[i];
    std::vector<uint32_t> cc((size_t)(A.nnz > 0 ? A.nnz : 0));
    for (int i = 0; i < A.nnz; ++i) cc[i] = (uint32_t)A.cols[i];
    return (host_only ? cutespmm_plan_build_host : cutespmm_plan_create)(plan, (uint64_t)A.nrows, (uint64_t)A.ncols, rp.data(), cc.data(),
                                                                          A.values, opts);
}
