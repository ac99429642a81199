// cpp_caller.cpp -- a C++ caller written against include/ozaki2.hpp exactly as the reference's programs are written against
// src/ozaki2.cuh (bench/ozaki_test.cu:66-73 of the reference: plan, dgemm, release on device arrays). Built and run by
// tests/test_gpu_api_surface.py with g++ (no nvcc: the header is plain C++ over the C ABI).
// usage: cpp_caller M N K nm in_A.bin in_B.bin out_C.bin
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_runtime.h>
#include "ozaki2.hpp"

static std::vector<double> load(const char *path, size_t n) {
    std::vector<double> v(n);
    FILE *f = fopen(path, "rb");
    if (!f || fread(v.data(), 8, n, f) != n) { fprintf(stderr, "cannot read %s\n", path); exit(2); }
    fclose(f);
    return v;
}

int main(int argc, char **argv) {
    if (argc != 8) return 2;
    const int M = atoi(argv[1]), N = atoi(argv[2]), K = atoi(argv[3]), nm = atoi(argv[4]);
    std::vector<double> A = load(argv[5], (size_t)M * K), B = load(argv[6], (size_t)K * N), C((size_t)M * N);
    double *dA, *dB, *dC;
    if (cudaMalloc(&dA, A.size() * 8) || cudaMalloc(&dB, B.size() * 8) || cudaMalloc(&dC, C.size() * 8)) return 3;
    cudaMemcpy(dA, A.data(), A.size() * 8, cudaMemcpyHostToDevice);
    cudaMemcpy(dB, B.data(), B.size() * 8, cudaMemcpyHostToDevice);
    oz::Plan p = oz::plan(M, N, K, nm);
    if (p.error) { fprintf(stderr, "plan: %s\n", ozb_error(p.error)); return 4; }
    if (p.bits != oz::bits_for(nm, K)) return 5;
    if (int e = oz::dgemm(p, dA, dB, dC)) { fprintf(stderr, "dgemm: %s\n", ozb_error(e)); return 6; }
    if (cudaDeviceSynchronize()) return 7;
    cudaMemcpy(C.data(), dC, C.size() * 8, cudaMemcpyDeviceToHost);
    oz::release(p);
    FILE *f = fopen(argv[7], "wb");
    fwrite(C.data(), 8, C.size(), f);
    fclose(f);
    printf("ok %s\n", ozb_version());
    return 0;
}
