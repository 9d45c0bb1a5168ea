/* rfk_io: the files either side of the render path - weights in, images out - behind a C ABI.
 *
 * Mirrors the reference's src/io (BANANASJIM/renderformer-cuda): SafeTensorsFile (safetensors.h:10-32,
 * safetensors.cpp:47-149), write_exr / write_png / tonemap_agx (image_writer.h:8-15, image_writer.cpp:17-72).
 * Differences in kind, not in meaning: the reader validates the header it parses (offsets inside the file, byte
 * sizes that match dtype x shape, every safetensors dtype named) instead of trusting it; the upload to the GPU goes
 * through two pinned staging buffers so that reading the file and the host-to-device copies overlap; the EXR and
 * PNG writers are written here against the formats' specifications (scan-line OpenEXR, FLOAT channels; zlib only for
 * the PNG's deflate stream) instead of through tinyexr / stb. The HDF5 scene reader (hdf5_reader.cpp:78-97) has no
 * counterpart: libhdf5 is not available to this build; a scene is five named arrays and travels in a safetensors
 * file with the keys of rf::Scene (triangles, texture, vn, c2w, fov) instead.
 *
 * Conventions: int status (0 ok, negative RFK_E* of rfk.h, positive cudaError_t); no exceptions cross the ABI;
 * strings are NUL-terminated UTF-8; host pointers unless the name says device.
 */
#ifndef RFK_IO_H
#define RFK_IO_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* rfk_stream_t; /* cudaStream_t */

/* Also declared in rfk.h with the same values. */
#ifndef RFK_OK
#define RFK_OK 0
#define RFK_EINVAL (-1)
#define RFK_EUNSUPPORTED (-2)
#endif
#define RFK_EIO (-10)     /* file cannot be opened, read, mapped or written */
#define RFK_EFORMAT (-11) /* file contents violate the format */
#define RFK_ENOTFOUND (-12)

/* Element types of a safetensors file (the format's dtype strings). */
enum {
    RFK_DTYPE_F32 = 0, RFK_DTYPE_F16 = 1, RFK_DTYPE_BF16 = 2, RFK_DTYPE_F64 = 3, RFK_DTYPE_I64 = 4, RFK_DTYPE_I32 = 5,
    RFK_DTYPE_I16 = 6, RFK_DTYPE_I8 = 7, RFK_DTYPE_U8 = 8, RFK_DTYPE_BOOL = 9, RFK_DTYPE_U16 = 10, RFK_DTYPE_U32 = 11,
    RFK_DTYPE_U64 = 12, RFK_DTYPE_F8_E4M3 = 13, RFK_DTYPE_F8_E5M2 = 14
};

typedef struct rfk_safetensors rfk_safetensors;

typedef struct rfk_tensor_info {
    const char* name;       /* owned by the file object */
    int dtype;              /* RFK_DTYPE_* */
    int ndim;
    const int64_t* shape;   /* ndim entries, owned by the file object */
    size_t offset;          /* byte offset inside the data section */
    size_t bytes;
    const void* host;       /* the tensor's bytes in the mapped file */
} rfk_tensor_info;

/* Maps the file and parses its header: 8-byte little-endian header length, JSON object of
 * name -> {dtype, shape, data_offsets}, optional "__metadata__" (kept, see rfk_safetensors_metadata).
 * replaces rf::SafeTensorsFile::load up to its upload — src/io/safetensors.cpp:47-136 */
int rfk_safetensors_open(const char* path, rfk_safetensors** out);
int rfk_safetensors_close(rfk_safetensors* f);
/* Number of tensors; entries are ordered by their offset in the data section. */
int rfk_safetensors_count(const rfk_safetensors* f);
int rfk_safetensors_entry(const rfk_safetensors* f, int index, rfk_tensor_info* info);
/* replaces rf::SafeTensorsFile::get / has — src/io/safetensors.cpp:138-149, safetensors.h:31 */
int rfk_safetensors_find(const rfk_safetensors* f, const char* name, rfk_tensor_info* info);
/* Size of the data section (what rfk_safetensors_upload copies). */
size_t rfk_safetensors_data_bytes(const rfk_safetensors* f);
/* Value of a "__metadata__" entry, or NULL. */
const char* rfk_safetensors_metadata(const rfk_safetensors* f, const char* key);
/* Copies the whole data section to device memory (device_dst: rfk_safetensors_data_bytes() bytes) in order, through
 * two pinned staging buffers, on `stream`; returns when the last copy has been enqueued and the staging buffers
 * are no longer needed (it synchronises the stream once at the end). A tensor then lives at device_dst + offset.
 * replaces the bulk upload of rf::SafeTensorsFile::load — src/io/safetensors.cpp:131-133 */
int rfk_safetensors_upload(const rfk_safetensors* f, void* device_dst, rfk_stream_t stream);

/* Writes a safetensors file from host arrays (the scene container and the tests use it; the reference only reads).
 * names / dtypes / ndims / shapes / data are arrays of n entries; shapes[i] has ndims[i] entries. */
int rfk_safetensors_write(const char* path, int n, const char* const* names, const int* dtypes, const int* ndims,
                          const int64_t* const* shapes, const void* const* data);

/* Interleaved [height][width][channels] fp32 -> OpenEXR, scan lines, FLOAT channels named B, G, R (A), no compression;
 * channels = 1 (written as Y), 3 or 4.
 * replaces rf::write_exr — src/io/image_writer.cpp:17-55 */
int rfk_write_exr(const char* path, const float* data, int width, int height, int channels);
/* Interleaved 8-bit image -> PNG (channels 1, 2, 3 or 4: grey, grey + alpha, RGB, RGBA), deflate through zlib.
 * replaces rf::write_png — src/io/image_writer.cpp:57-59 */
int rfk_write_png(const char* path, const unsigned char* data, int width, int height, int channels);
/* HDR -> LDR: v = max(v, 0); v = v / (v + 1); v = v^(1/2.2); byte = clamp(v * 255, 0, 255) truncated.
 * replaces rf::tonemap_agx — src/io/image_writer.cpp:61-72 */
int rfk_tonemap(const float* hdr, unsigned char* ldr, int width, int height, int channels);

#ifdef __cplusplus
}
#endif
#endif /* RFK_IO_H */
