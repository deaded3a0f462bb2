// Kernel-parameter rows: the 11-column CSV format of the reference
// (readme.md:46-60; read by include/utils/readCSV.h:13-33 and consumed at
// main.cu:8-32 and fft_codegen.py:745-752):
//   logN, launches, logN1, logN2, logN3, BS1, BS2, BS3, n1, n2, n3
// logNi = log2 of the sub-transform of launch i, BSi = lines per thread block,
// ni = points per thread.  Row r of the file describes logN = r, as in the reference.
#pragma once
#include <string>
#include <vector>

namespace tfft {

struct ParamRow {
    int logn = 0;
    int launches = 0;
    int logni[3] = {0, 0, 0};
    int bs[3] = {0, 0, 0};
    int n[3] = {0, 0, 0};
};

// Parses CSV text; rows are indexed by their first column.  Returns false and
// fills err on a malformed line.
bool parse_param_csv(const std::string& text, std::vector<ParamRow>& rows, std::string& err);
bool load_param_file(const std::string& path, std::vector<ParamRow>& rows, std::string& err);
// Built-in B200 table (generated from param/B200/param_<dtype>.csv at build time).
const char* builtin_param_csv(int dtype);
// Structural checks shared by the planner and the tests: 1..3 launches, sizes add
// up to logN, BS and n powers of two, n <= 32.
bool validate_row(const ParamRow& r, std::string& err);
// Built-in single-pass table (param/B200/single_pass_<dtype>.csv, lines "logN, log2 cluster
// size"): log2 of the cluster size the size logN runs with as one cluster kernel, or -1 if
// the size is not in the table and runs the launches of its parameter row.
int builtin_single_pass_cluster(int dtype, int logn);
// Built-in thread_bs table (param/B200/thread_bs_<dtype>.csv, lines "logN, FT off, FT on"): what a
// plan created with thread_bs = 0 uses; 1 for sizes that are not listed.
int builtin_thread_bs(int dtype, int logn, int ft);

}  // namespace tfft
