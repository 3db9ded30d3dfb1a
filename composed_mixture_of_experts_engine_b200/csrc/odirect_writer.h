// C interface of the checkpoint file writer (odirect_writer.cpp).
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// Writes `n` bytes at `data` to `path` (created/truncated), then fsyncs.  With use_odirect != 0 the file is
// opened with O_DIRECT and written from a page-aligned bounce buffer in `chunk_bytes` pieces (the unaligned
// tail is written through a second, buffered descriptor); if the filesystem refuses O_DIRECT the call falls
// back to buffered writes.  Returns 0 on success, otherwise errno.  *used_odirect (optional) reports whether
// the direct path was taken.
int cmoe_write_file(const char* path, const void* data, size_t n, int use_odirect, size_t chunk_bytes,
                    int* used_odirect);

#ifdef __cplusplus
}
#endif
