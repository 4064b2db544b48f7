// Batch loader over a device-resident dataset: the index bookkeeping of the reference's DataLoader
// (src/dataset.zig:121-223) on the host, the per-batch copy as one gather kernel on the device.
//
// The images (fp32, num_samples x input_dim) and labels (u8) live in device memory for the loader's lifetime;
// the sample order lives in a host vector (shuffled exactly as the reference shuffles it) with a device copy
// refreshed once per epoch, so next_into() is a single kernel launch and moves no host data.
#include <stdint.h>
#include <stdio.h>

#include <algorithm>
#include <memory>
#include <numeric>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../../include/znn_cuda.h"
#include "../../../include/znn_host.h"

namespace znn {
int fail(int code, const char* fmt, ...);  // runtime.cu: sets the thread's error text
}

namespace {

// std.Random.DefaultPrng of the reference's toolchain: xoshiro256++ seeded through SplitMix64.
struct Xoshiro256 {
    uint64_t s[4];
    explicit Xoshiro256(uint64_t seed)
    {
        uint64_t x = seed;
        for (auto& w : s) {
            x += 0x9e3779b97f4a7c15ull;
            uint64_t z = x;
            z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
            z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
            w = z ^ (z >> 31);
        }
    }
    static uint64_t rotl(uint64_t v, int k) { return (v << k) | (v >> (64 - k)); }
    uint64_t next()
    {
        const uint64_t r = rotl(s[0] + s[3], 23) + s[0];
        const uint64_t t = s[1] << 17;
        s[2] ^= s[0];
        s[3] ^= s[1];
        s[1] ^= s[2];
        s[0] ^= s[3];
        s[2] ^= t;
        s[3] = rotl(s[3], 45);
        return r;
    }
    // uniform in [0, less_than): Lemire's multiply-and-reject, as std.Random.uintLessThan(u64, ...) draws it
    uint64_t below(uint64_t less_than)
    {
        unsigned __int128 m = (unsigned __int128)next() * less_than;
        uint64_t l = (uint64_t)m;
        if (l < less_than) {
            uint64_t t = 0 - less_than;
            if (t >= less_than) {
                t -= less_than;
                if (t >= less_than) t %= less_than;
            }
            while (l < t) {
                m = (unsigned __int128)next() * less_than;
                l = (uint64_t)m;
            }
        }
        return (uint64_t)(m >> 64);
    }
};

// whole file into memory; empty vector + false on any I/O error
bool read_file(const char* path, std::vector<uint8_t>& out)
{
    FILE* f = fopen(path, "rb");
    if (!f) return false;
    uint8_t chunk[65536];
    size_t got;
    while ((got = fread(chunk, 1, sizeof chunk, f)) > 0) out.insert(out.end(), chunk, chunk + got);
    const bool ok = !ferror(f);
    fclose(f);
    return ok;
}

uint32_t be32(const uint8_t* p) { return (uint32_t)p[0] << 24 | (uint32_t)p[1] << 16 | (uint32_t)p[2] << 8 | p[3]; }

}  // namespace

struct znn_loader {
    const float* images = nullptr;
    const uint8_t* labels = nullptr;
    size_t num_samples = 0;
    int input_dim = 0;
    size_t batch_size = 0;
    bool shuffle = false, drop_last = false;
    std::vector<int32_t> indices;
    int32_t* d_indices = nullptr;
    size_t current_index = 0;
    Xoshiro256 prng{1337};

    // src/dataset.zig:166-175: Fisher-Yates from the top, j drawn from [0, i]
    void shuffle_indices()
    {
        for (size_t i = indices.size() - 1; i > 0; --i) {
            const size_t j = (size_t)prng.below((uint64_t)i + 1);
            std::swap(indices[i], indices[j]);
        }
    }
    int upload_order()
    {
        if (indices.empty()) return ZNN_OK;
        return znn_memcpy_h2d(d_indices, indices.data(), indices.size() * sizeof(int32_t));
    }
    // src/dataset.zig:184-194
    size_t peek() const
    {
        if (current_index >= num_samples) return 0;
        const size_t remaining = num_samples - current_index;
        if (drop_last && remaining < batch_size) return 0;
        return remaining < batch_size ? remaining : batch_size;
    }
};

extern "C" {

// loadImages + loadLabels (src/dataset.zig:23-106) with the pixel conversion on the device: the IDX files are
// read on the host, the pixel bytes go up once, and pixel / 255 is computed there into the fp32 image matrix.
int znn_dataset_load_idx(const char* images_path, const char* labels_path, float** images, uint8_t** labels,
                         unsigned* num_images, unsigned* rows, unsigned* cols, unsigned* num_labels)
{
    if (!images_path || !labels_path || !images || !labels || !num_images || !rows || !cols || !num_labels)
        return znn::fail(ZNN_ERR_INVALID, "NULL argument");
    *images = nullptr;
    *labels = nullptr;
    std::vector<uint8_t> img, lab;
    if (!read_file(images_path, img)) return znn::fail(ZNN_ERR_INVALID, "cannot read %s", images_path);
    if (!read_file(labels_path, lab)) return znn::fail(ZNN_ERR_INVALID, "cannot read %s", labels_path);
    if (img.size() < 16) return znn::fail(ZNN_ERR_INVALID, "%s: EndOfStream in the header", images_path);
    if (be32(img.data()) != 0x00000803u) return znn::fail(ZNN_ERR_INVALID, "%s: InvalidMagicNumber", images_path);
    const uint32_t n = be32(img.data() + 4), r = be32(img.data() + 8), c = be32(img.data() + 12);
    const size_t per_image = (size_t)r * c;   // < 2^64: two 32-bit factors
    if (n != 0 && per_image > (size_t)-1 / n) return znn::fail(ZNN_ERR_INVALID, "%s: implausible header", images_path);
    const size_t num_pixels = per_image * n;
    if (img.size() - 16 < num_pixels) return znn::fail(ZNN_ERR_INVALID, "%s: EndOfStream in the pixels", images_path);
    if (lab.size() < 8) return znn::fail(ZNN_ERR_INVALID, "%s: EndOfStream in the header", labels_path);
    if (be32(lab.data()) != 0x00000801u) return znn::fail(ZNN_ERR_INVALID, "%s: InvalidMagicNumber", labels_path);
    const uint32_t items = be32(lab.data() + 4);
    if (lab.size() - 8 < items) return znn::fail(ZNN_ERR_INVALID, "%s: EndOfStream in the labels", labels_path);

    float* d_img = nullptr;
    uint8_t *d_lab = nullptr, *d_px = nullptr;
    int rc = ZNN_OK;
    auto step = [&](int code) { if (rc == ZNN_OK) rc = code; };
    step(znn_malloc((void**)&d_img, std::max<size_t>(num_pixels, 1) * sizeof(float)));
    step(znn_malloc((void**)&d_lab, std::max<size_t>(items, 1)));
    step(znn_malloc((void**)&d_px, std::max<size_t>(num_pixels, 1)));
    if (rc == ZNN_OK && num_pixels) step(znn_memcpy_h2d(d_px, img.data() + 16, num_pixels));
    if (rc == ZNN_OK && items) step(znn_memcpy_h2d(d_lab, lab.data() + 8, items));
    if (rc == ZNN_OK) step(znn_pixels_to_unit(d_px, d_img, num_pixels));
    if (rc == ZNN_OK) step(znn_sync());
    if (d_px) znn_free(d_px);
    if (rc != ZNN_OK) {
        if (d_img) znn_free(d_img);
        if (d_lab) znn_free(d_lab);
        return rc;
    }
    *images = d_img;
    *labels = d_lab;
    *num_images = n;
    *rows = r;
    *cols = c;
    *num_labels = items;
    return ZNN_OK;
}

int znn_loader_create(const float* images, const uint8_t* labels, size_t num_samples, int input_dim, size_t batch_size,
                      int shuffle, int drop_last, long long seed, znn_loader** out)
{
    if (!out) return znn::fail(ZNN_ERR_INVALID, "out is NULL");
    *out = nullptr;
    if (!images || !labels) return znn::fail(ZNN_ERR_INVALID, "images/labels is NULL");
    if (num_samples == 0 || num_samples > 0x7fffffffull) return znn::fail(ZNN_ERR_INVALID, "num_samples must be 1..2^31-1");
    if (input_dim <= 0) return znn::fail(ZNN_ERR_INVALID, "input_dim must be positive");
    if (batch_size == 0 || batch_size > 65535) return znn::fail(ZNN_ERR_INVALID, "batch_size must be 1..65535");
    std::unique_ptr<znn_loader> l(new znn_loader);
    l->images = images;
    l->labels = labels;
    l->num_samples = num_samples;
    l->input_dim = input_dim;
    l->batch_size = batch_size;
    l->shuffle = shuffle != 0;
    l->drop_last = drop_last != 0;
    l->indices.resize(num_samples);
    std::iota(l->indices.begin(), l->indices.end(), 0);
    l->prng = Xoshiro256(seed < 0 ? 1337ull : (uint64_t)seed);   // options.seed orelse 1337 (src/dataset.zig:155)
    int rc = znn_malloc((void**)&l->d_indices, num_samples * sizeof(int32_t));
    if (rc != ZNN_OK) return rc;
    if (l->shuffle) l->shuffle_indices();
    rc = l->upload_order();
    if (rc != ZNN_OK) {
        znn_free(l->d_indices);
        return rc;
    }
    *out = l.release();
    return ZNN_OK;
}

int znn_loader_destroy(znn_loader* l)
{
    if (!l) return ZNN_OK;
    znn_sync();
    if (l->d_indices) znn_free(l->d_indices);
    delete l;
    return ZNN_OK;
}

// src/dataset.zig:177-182
int znn_loader_reset(znn_loader* l)
{
    if (!l) return znn::fail(ZNN_ERR_INVALID, "loader is NULL");
    l->current_index = 0;
    if (l->shuffle) {
        l->shuffle_indices();
        return l->upload_order();
    }
    return ZNN_OK;
}

int znn_loader_set_drop_last(znn_loader* l, int drop_last)
{
    if (!l) return znn::fail(ZNN_ERR_INVALID, "loader is NULL");
    l->drop_last = drop_last != 0;
    return ZNN_OK;
}

int znn_loader_peek_next_batch_size(znn_loader* l, size_t* n)
{
    if (!l || !n) return znn::fail(ZNN_ERR_INVALID, "loader/n is NULL");
    *n = l->peek();
    return ZNN_OK;
}

// src/dataset.zig:197-222; *n = 0 where the reference returns null
int znn_loader_next_into(znn_loader* l, float* x_dest, uint8_t* y_dest, size_t* n)
{
    if (!l || !n) return znn::fail(ZNN_ERR_INVALID, "loader/n is NULL");
    *n = 0;
    const size_t take = l->peek();
    if (take == 0) return ZNN_OK;
    if (!x_dest || !y_dest) return znn::fail(ZNN_ERR_INVALID, "x_dest/y_dest is NULL");
    const int rc = znn_batch_gather(l->images, l->labels, l->d_indices + l->current_index, x_dest, y_dest, (int)take,
                                    l->input_dim, l->num_samples);
    if (rc != ZNN_OK) return rc;
    l->current_index += take;
    *n = take;
    return ZNN_OK;
}

int znn_loader_indices(znn_loader* l, int32_t* host_out, size_t count)
{
    if (!l || !host_out) return znn::fail(ZNN_ERR_INVALID, "loader/host_out is NULL");
    if (count != l->indices.size()) return znn::fail(ZNN_ERR_INVALID, "count must equal the number of samples");
    std::copy(l->indices.begin(), l->indices.end(), host_out);
    return ZNN_OK;
}

}  // extern "C"
