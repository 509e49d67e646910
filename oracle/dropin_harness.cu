// dropin_harness.cu -- runs the reference project's OWN flash-attention smokes with this repository's kernels behind them.
//
// THIS FILE IS TEST INFRASTRUCTURE.  oracle/Makefile links it with the reference's unmodified
// sentinel/NeuralNet/Cuda/{CudaCausalSelfAttention,CudaMatmul,CudaOps,CudaAmp,CudaAdam,CudaKvCache}.cu and the host
// sources they need, but with sentinel_b200/csrc/sentinel_compat.cu (built with -DSNTL_COMPAT_USE_SENTINEL_TYPES) in
// the place of sentinel/NeuralNet/Cuda/CudaFlashAttention.cu, and against libsntl_attn.so.  The reference's attention
// layer then reaches this library through its two unmodified launch sites (CudaCausalSelfAttention.cu:237-249, :421-438).
//
//   dropin_smoke flash <embed> <heads> <seq> <maxpos>   CudaCausalSelfAttention::runFlashParitySmokeDemo
//                                                       (CudaCausalSelfAttention.cu:817-894; called with (64,4,48,64),
//                                                       (768,12,128,512), (768,12,256,512), (768,12,1024,1024) at
//                                                       sentinel/main.cpp:640-643); it throws when the flash path was
//                                                       not taken and prints flash-versus-dense differences
//   dropin_smoke gqa                                    CudaCausalSelfAttention::runGqaCudaSmokeDemo (:896-997); it
//                                                       throws when flash and dense differ by more than 1e-3 / 1e-1
//
// Built with -DSNTL_HARNESS_REFERENCE and the reference's own CudaFlashAttention.cu (oracle/_ref/dropin_smoke_reference)
// the same harness runs the reference's smokes on the reference's kernels: the figures to read the above against.
//
// After the smoke the harness prints which kernel family of this library ran (`path=`), how many of its kernels were
// launched (`launches=`) and the device status poll (`device_status=`).  Exit code 0 = the smoke returned normally and
// this library's kernels ran; 1 = it threw; 2 = usage; 3 = the smoke passed without a launch from this library;
// 4 = no CUDA device (the reference's smokes print "skipped" and nothing is computed).
#include "NeuralNet/Cuda/CudaCausalSelfAttention.hpp"
#include "NeuralNet/Cuda/CudaFlashAttention.hpp"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>

#ifndef SNTL_HARNESS_REFERENCE
#include "sentinel_compat.hpp"
#include "sntl_attn.h"
#endif

int main(int argc, char** argv)
{
    if (argc < 2) {
        std::fprintf(stderr, "usage: %s flash <embed> <heads> <seq> <maxpos> | gqa\n", argv[0]);
        return 2;
    }
    std::printf("maxHeadDimension=%d\n", CudaFlashAttention::maxHeadDimension);
    if (!CudaMatmul::isAvailable()) {
        std::printf("no CUDA device\n");
        return 4;
    }
#ifndef SNTL_HARNESS_REFERENCE
    const unsigned long long before = (unsigned long long)sntl_attn_launch_count();
#endif
    try {
        if (std::strcmp(argv[1], "flash") == 0 && argc == 6) {
            CudaCausalSelfAttention::runFlashParitySmokeDemo(std::atoi(argv[2]), std::atoi(argv[3]), std::atoi(argv[4]),
                                                             std::atoi(argv[5]));
        } else if (std::strcmp(argv[1], "gqa") == 0) {
            CudaCausalSelfAttention::runGqaCudaSmokeDemo();
        } else {
            std::fprintf(stderr, "unknown mode\n");
            return 2;
        }
#ifndef SNTL_HARNESS_REFERENCE
        sentinel_b200::throwIfDeviceWaitTimedOut();
#endif
    } catch (const std::exception& e) {
        std::fflush(stdout);
        std::printf("threw=%s\n", e.what());
        return 1;
    }
#ifdef SNTL_HARNESS_REFERENCE
    std::printf("path=reference\n");
    return 0;
#else
    const unsigned long long launches = (unsigned long long)sntl_attn_launch_count() - before;
    std::printf("path=%s\nlaunches=%llu\ndevice_status=ok\n", sentinel_b200::lastPath(), launches);
    return launches > 0 ? 0 : 3;
#endif
}
