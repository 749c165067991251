// Launch entry points of the manifold-convolution kernels.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace chop {
struct ScArgs;
int sc_fwd_simt_launch(int dtype, const ScArgs& a, cudaStream_t st);
int sc_dgrad_simt_launch(int dtype, const ScArgs& a, cudaStream_t st);
int sc_wgrad_simt_launch(int dtype, const ScArgs& a, cudaStream_t st);
int sc_tconv_simt_launch(int dtype, const ScArgs& a, cudaStream_t st);
int sc_twgrad_simt_launch(int dtype, const ScArgs& a, int nparts, cudaStream_t st);
int sc_pad_launch(int dtype, bool grad, const void* src, const int* base_plane, void* dst, int B, int h, int w, int d,
                  int C, int sr, int sc, int sd, cudaStream_t st);
int sc_wgrad_parts(long long nvox_out);
int sc_wgrad_simt_launch_parts(int dtype, const ScArgs& a, int nparts, cudaStream_t st);
int sc_static_scratch(void** ptr, size_t* bytes);
bool sc_umma_supported(int dtype, const ScArgs& a);
int sc_umma_fwd_launch(const ScArgs& a, cudaStream_t st);
int sc_umma_dgrad_launch(const ScArgs& a, cudaStream_t st);
int sc_umma_wgrad_launch(const ScArgs& a, int nparts, cudaStream_t st);
int sc_umma_twgrad_launch(const ScArgs& a, int nparts, cudaStream_t st);
bool sc_tile_supported(int dtype, const ScArgs& a);
int sc_tile_fwd_launch(int dtype, const ScArgs& a, cudaStream_t st);
bool sc_tile_wgrad_supported(int dtype, const ScArgs& a, bool transposed);
int sc_tile_wgrad_launch(int dtype, const ScArgs& a, int nparts, cudaStream_t st);
int sc_tile_twgrad_launch(int dtype, const ScArgs& a, int nparts, cudaStream_t st);
int sc_tile_gather_launch(int dtype, const ScArgs& a, cudaStream_t st);
int sc_umma_timeouts();
int sc_umma_watch();
int sc_umma_note_timeout_for_test(int on);
void sc_umma_set_rows(int on);
size_t sc_wgrad_workspace_bytes(int dtype, int taps, int Cin, int Cout, long long nvox_out);
}  // namespace chop
