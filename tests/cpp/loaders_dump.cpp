// Reads a MatrixMarket file with SparseCoo, converts it with CSR_Matrix (include/cutespmm_loaders.hpp)
// and prints the CSR arrays, one array per line, so a test can compare them with what the
// reference's loaders produced for the same file.  Also exercises the small surface around them
// (Insert_Next, DenseToCSR/ToDense round trip, save_mtx, SMA, the host-only plan bridge).
#include <cstdio>
#include <string>

#include "cutespmm_loaders.hpp"

int main(int argc, char **argv)
{
    if (argc < 2) return 2;
    SparseCoo<float> coo{std::string(argv[1])};
    CSR_Matrix<float> csr(coo);
    std::printf("%d %d %d\n", csr.nrows, csr.ncols, csr.nnz);
    for (int i = 0; i <= csr.nrows; ++i) std::printf("%d ", csr.rowPtr[i]);
    std::printf("\n");
    for (int i = 0; i < csr.nnz; ++i) std::printf("%d ", csr.cols[i]);
    std::printf("\n");
    for (int i = 0; i < csr.nnz; ++i) std::printf("%.9g ", csr.values[i]);
    std::printf("\n");

    int bad = 0;
    // dense round trip
    std::vector<float> dense = csr.ToDense();
    CSR_Matrix<float> again(dense.data(), csr.nrows, csr.ncols);
    std::vector<float> dense2 = again.ToDense();
    bad += dense != dense2;
    // save / reload keeps the coordinate list
    if (argc > 2) {
        coo.save_mtx(argv[2]);
        SparseCoo<float> back{std::string(argv[2])};
        bad += back.data_vector.size() != coo.data_vector.size();
        for (size_t i = 0; i < back.data_vector.size() && !bad; ++i)
            bad += back.data_vector[i].row != coo.data_vector[i].row || back.data_vector[i].col != coo.data_vector[i].col;
    }
    // Insert_Next + prepare_for_cusparse
    SparseCoo<float> made(3, 3, 0);
    made.Insert_Next(2, 1, 5.f);
    made.Insert_Next(0, 0, 1.f);
    made.prepare_for_cusparse();
    bad += made.nnz != 2 || made.rows[0] != 2 || made.values[1] != 1.f;
    CSR_Matrix<float> m2(made);
    bad += m2.rowPtr[1] != 1 || m2.rowPtr[3] != 2 || m2.cols[1] != 1;
    // moving average over a window of 3
    SMA sma(3);
    for (double v : {3.0, 6.0, 9.0, 12.0}) sma.add(v);
    bad += sma.avg() != 9.0;
    // bridge to the library (host-only plan: no GPU needed)
    cutespmm_plan_t *plan = nullptr;
    bad += cutespmm_plan_from_csr(&plan, csr, nullptr, true) != CUTESPMM_OK;
    cutespmm_plan_info_t info;
    bad += cutespmm_plan_info(plan, &info) != CUTESPMM_OK || (int)info.nnz != csr.nnz;
    cutespmm_plan_destroy(plan);
    std::printf("selfcheck %s\n", bad ? "FAILED" : "ok");
    return bad ? 1 : 0;
}
