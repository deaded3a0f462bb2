#include "params.h"

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>

namespace tfft {

static bool is_pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }

bool parse_param_csv(const std::string& text, std::vector<ParamRow>& rows, std::string& err) {
    rows.clear();
    std::istringstream ss(text);
    std::string line;
    int lineno = 0;
    while (std::getline(ss, line)) {
        ++lineno;
        if (line.find_first_not_of(" \t\r\n") == std::string::npos) continue;
        if (line[line.find_first_not_of(" \t")] == '#') continue;
        std::vector<long long> tok;
        std::istringstream ls(line);
        std::string cell;
        while (std::getline(ls, cell, ',')) {
            char* end = nullptr;
            long long v = std::strtoll(cell.c_str(), &end, 10);
            if (end == cell.c_str()) {
                err = "line " + std::to_string(lineno) + ": not a number: '" + cell + "'";
                return false;
            }
            tok.push_back(v);
        }
        if (tok.size() != 11) {
            err = "line " + std::to_string(lineno) + ": expected 11 columns, got " + std::to_string(tok.size());
            return false;
        }
        ParamRow r;
        r.logn = (int)tok[0];
        r.launches = (int)tok[1];
        for (int i = 0; i < 3; ++i) {
            r.logni[i] = (int)tok[2 + i];
            r.bs[i] = (int)tok[5 + i];
            r.n[i] = (int)tok[8 + i];
        }
        if (r.logn < 0 || r.logn > 40) {
            err = "line " + std::to_string(lineno) + ": logN out of range";
            return false;
        }
        if ((int)rows.size() <= r.logn) rows.resize(r.logn + 1);
        rows[r.logn] = r;
    }
    return true;
}

bool load_param_file(const std::string& path, std::vector<ParamRow>& rows, std::string& err) {
    std::ifstream f(path.c_str());
    if (!f.is_open()) {
        err = "cannot open " + path;
        return false;
    }
    std::stringstream buf;
    buf << f.rdbuf();
    return parse_param_csv(buf.str(), rows, err);
}

bool validate_row(const ParamRow& r, std::string& err) {
    if (r.launches < 1 || r.launches > 3) {
        err = "launches must be 1..3";
        return false;
    }
    int sum = 0;
    for (int i = 0; i < r.launches; ++i) {
        if (r.logni[i] < 1) {
            err = "logNi must be >= 1";
            return false;
        }
        if (!is_pow2(r.bs[i]) || !is_pow2(r.n[i]) || r.n[i] < 2 || r.n[i] > 32) {
            err = "BSi and ni must be powers of two, 2 <= ni <= 32";
            return false;
        }
        sum += r.logni[i];
    }
    if (sum != r.logn) {
        err = "logN1+logN2+logN3 != logN";
        return false;
    }
    return true;
}

static const char* k_builtin_float2 =
#include "generated/default_params_float2.inc"
    ;
static const char* k_builtin_double2 =
#include "generated/default_params_double2.inc"
    ;

const char* builtin_param_csv(int dtype) { return dtype == 0 ? k_builtin_float2 : k_builtin_double2; }

static const char* k_single_pass_float2 =
#include "generated/default_single_pass_float2.inc"
    ;
static const char* k_single_pass_double2 =
#include "generated/default_single_pass_double2.inc"
    ;

static const char* k_thread_bs_float2 =
#include "generated/default_thread_bs_float2.inc"
    ;
static const char* k_thread_bs_double2 =
#include "generated/default_thread_bs_double2.inc"
    ;

int builtin_thread_bs(int dtype, int logn, int ft) {
    std::istringstream ss(dtype == 0 ? k_thread_bs_float2 : k_thread_bs_double2);
    std::string line;
    while (std::getline(ss, line)) {
        int l = -1, off = 1, on = 1;
        if (sscanf(line.c_str(), "%d , %d , %d", &l, &off, &on) == 3 && l == logn) {
            const int v = ft ? on : off;
            return v >= 1 ? v : 1;
        }
    }
    return 1;
}

int builtin_single_pass_cluster(int dtype, int logn) {
    std::istringstream ss(dtype == 0 ? k_single_pass_float2 : k_single_pass_double2);
    std::string line;
    while (std::getline(ss, line)) {
        if (line.find_first_not_of(" \t\r\n") == std::string::npos || line[line.find_first_not_of(" \t")] == '#') continue;
        int l = -1, g = -1;
        if (sscanf(line.c_str(), "%d , %d", &l, &g) == 2 && l == logn) return g;
    }
    return -1;
}

}  // namespace tfft
