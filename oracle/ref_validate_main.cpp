// TEST INFRASTRUCTURE ONLY. Command-line front end to the reference's own generated host contract
// (tests/gpu/generated/fmha_fwd_hd128_mxfp8_v3_*_abi.h of the reference tree, included from where it lies, against the stub HIP
// runtime): reads cases from stdin, one per line,
//     <kernel 0..3> <hex of the packed Args> <10 buffer sizes> <grid x y z> <B HK KL>
// and prints per case "1" (valid) or "0 <message>" as the reference's validate() reports it. Used to check the C ABI's
// fmha_mxfp8_validate against the reference byte for byte, and to produce tests/golden/validate_cases.json.
#include <hip/hip_runtime.h>
#include "generated/shipped_abi.h"

#include <iostream>
#include <sstream>
#include <string>
#include <vector>

namespace hg = amdc_hostgen;

template <class NS_Args>
static bool load(const std::string& hex, NS_Args& a) {
    if (hex.size() != 2 * sizeof(NS_Args)) return false;
    unsigned char* p = reinterpret_cast<unsigned char*>(&a);
    for (size_t i = 0; i < sizeof(NS_Args); ++i) p[i] = (unsigned char)std::stoi(hex.substr(2 * i, 2), nullptr, 16);
    return true;
}

int main() {
    std::string line;
    while (std::getline(std::cin, line)) {
        std::istringstream is(line);
        int kernel; std::string hex; uint64_t sz[10]; unsigned g[3]; long long B, HK, KL;
        is >> kernel >> hex;
        for (auto& s : sz) is >> s;
        is >> g[0] >> g[1] >> g[2] >> B >> HK >> KL;
        std::string err; bool ok = false;
        if (kernel == 0) {
            namespace K = hg::fmha_fwd_hd128_mxfp8_v3_vs128;
            K::Args a{}; if (!load(hex, a)) { std::cout << "0 bad-size\n"; continue; }
            K::BufferSizes b{}; b.ptr_q = sz[0]; b.ptr_k = sz[1]; b.ptr_v = sz[2]; b.ptr_o = sz[3]; b.ptr_q_descale = sz[4]; b.ptr_k_descale = sz[5]; b.ptr_v_descale = sz[6];
            K::Symbols s{}; s.HK = HK;
            ok = K::validate(a, b, dim3(g[0], g[1], g[2]), s, &err);
        } else if (kernel == 1) {
            namespace K = hg::fmha_fwd_hd128_mxfp8_v3_t128;
            K::Args a{}; if (!load(hex, a)) { std::cout << "0 bad-size\n"; continue; }
            K::BufferSizes b{}; b.ptr_q = sz[0]; b.ptr_k = sz[1]; b.ptr_v = sz[2]; b.ptr_o = sz[3]; b.ptr_q_descale = sz[4]; b.ptr_k_descale = sz[5]; b.ptr_v_descale = sz[6];
            K::Symbols s{}; s.HK = HK;
            ok = K::validate(a, b, dim3(g[0], g[1], g[2]), s, &err);
        } else if (kernel == 2) {
            namespace K = hg::fmha_fwd_hd128_mxfp8_v3_kvsplit;
            K::Args a{}; if (!load(hex, a)) { std::cout << "0 bad-size\n"; continue; }
            K::BufferSizes b{}; b.ptr_q = sz[0]; b.ptr_k = sz[1]; b.ptr_v = sz[2]; b.ptr_o = sz[3]; b.ptr_q_descale = sz[4]; b.ptr_k_descale = sz[5]; b.ptr_v_descale = sz[6];
            b.ptr_ohat = sz[7]; b.ptr_lse = sz[8];
            K::Symbols s{}; s.B = B; s.HK = HK; s.KL = KL;
            ok = K::validate(a, b, dim3(g[0], g[1], g[2]), s, &err);
        } else if (kernel == 3) {
            namespace K = hg::fmha_fwd_hd128_mxfp8_v3_kvsplit_combine8h;
            K::Args a{}; if (!load(hex, a)) { std::cout << "0 bad-size\n"; continue; }
            K::BufferSizes b{}; b.ptr_ohat = sz[7]; b.ptr_lse = sz[8]; b.ptr_out = sz[9];
            ok = K::validate(a, b, dim3(g[0], g[1], g[2]), K::Symbols{}, &err);
        } else { std::cout << "0 bad-kernel\n"; continue; }
        if (ok) std::cout << "1\n"; else std::cout << "0 " << err << "\n";
    }
    return 0;
}
