// shrike_sample_no_alloc: the sampling kernels for callers that must not allocate.
//
// This entry point has no counterpart in Azimml/shrike; it is an addition of this
// library.
//
// Who it is for.  `shrike_sample` needs a little scratch memory (the winner of every
// vocabulary slice of every row) and takes it from the caller, who normally gets it from
// an allocator.  Some callers cannot do that at the moment they sample: an engine that
// has already handed all free device memory to its key/value pool, so that cudaMalloc
// would fail; a step loop that must not hit cudaMalloc or cudaFree because either may
// synchronise the whole device and stall every stream; code that runs inside somebody
// else's memory manager and is forbidden to call an allocator at all.  For them the
// scratch lives in a fixed array inside the library's device image.
//
// The price and the limits.
//   * The array is SHRIKE_SAMPLE_NO_ALLOC_BYTES (256 KiB) of device memory on every GPU
//     that loads this library, held until the process exits.
//   * At most SHRIKE_SAMPLE_NO_ALLOC_MAX_ROWS rows per call; any vocabulary size.  More
//     rows are refused with SHRIKE_SAMPLE_NO_ALLOC_TOO_MANY_ROWS and nothing is launched;
//     `shrike_sample_no_alloc_message` turns a code into text.
//   * All calls share the one array.  It keeps what the last call left; that is harmless,
//     because every entry a call reads it has written itself first (nothing has to start
//     at zero).  Two calls that overlap on the GPU (different streams, or different
//     threads without ordering) race on it: serialise them.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current).  Make that first call outside any
//     stream capture.
//   * Devices with an index of 64 or more are refused (SHRIKE_SAMPLE_NO_ALLOC_BAD_DEVICE).
//   * A row whose logits are all NaN has no largest element; it yields token 0.
//   * No cudaMalloc, cudaFree or other allocating routine is called, on any call.
// The caller passes inputs and outputs exactly as for `shrike_sample`:
//   logits [rows, vocab] float32, temperature [rows] float32, top_p [rows] float32,
//   seeds [rows] int64, out [rows] int32, all device pointers; results are the same
//   tokens `shrike_sample` gives for the same inputs.
#pragma once
#include <cuda_runtime.h>

#define SHRIKE_SAMPLE_NO_ALLOC_MAX_ROWS 256
#define SHRIKE_SAMPLE_NO_ALLOC_MAX_SLICES 128
#define SHRIKE_SAMPLE_NO_ALLOC_BYTES (SHRIKE_SAMPLE_NO_ALLOC_MAX_ROWS * SHRIKE_SAMPLE_NO_ALLOC_MAX_SLICES * 8)
#define SHRIKE_SAMPLE_NO_ALLOC_TOO_MANY_ROWS (-2)
#define SHRIKE_SAMPLE_NO_ALLOC_BAD_DEVICE (-3)

extern "C" int shrike_sample_no_alloc(const float* logits, const float* temperature, const float* top_p,
                                      const long long* seeds, int* out, int rows, int vocab,
                                      cudaStream_t stream);
extern "C" const char* shrike_sample_no_alloc_message(int code);
