// Sharded token loader: the reference's DataLoader (src/train/data_loader.cpp) for data-parallel training.
//
// Same file format (a flat array of uint16 token ids), same sampling: samples are the seq_len-long windows at
// base_offset + i * seq_len (i < count / seq_len - 1), base_offset drawn per epoch in [0, seq_len), the windows shuffled with
// Fisher-Yates, both with the C library's rand() (the reference seeds it with srand(seed) in src/train/train.cpp:73).  A
// batch takes the next samples of that order; labels are the inputs shifted by one token.  With world = 1 the batches are the
// reference's batches.  With world > 1 a step consumes world * batch consecutive samples of the SAME order on every rank
// (every rank must have seeded rand() alike and drawn the same numbers), and rank r copies out samples [r * batch, (r + 1) *
// batch) of them: together the ranks see exactly the global batch that one process with batch world * batch would see.
// Host-only code; the caller copies the batch to its device (gptb200_memcpy_h2d or its own pinned staging).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/gptb200.h"

struct gptb200_loader {
    std::vector<int> data;
    std::vector<int> order;   // start token of every sample of this epoch, shuffled
    int seq_len = 0;
    size_t cursor = 0;        // samples consumed in this epoch (all ranks together)
};

extern "C" {

int gptb200_loader_create(gptb200_loader **out, const char *path, int seq_len)
{
    if (!out || !path || seq_len <= 0) return GPTB200_ERR_INVALID_ARG;
    *out = nullptr;
    FILE *fp = fopen(path, "rb");
    if (!fp) return GPTB200_ERR_INVALID_ARG;
    fseek(fp, 0, SEEK_END);
    const long bytes = ftell(fp);
    fseek(fp, 0, SEEK_SET);
    const size_t count = bytes > 0 ? size_t(bytes) / sizeof(uint16_t) : 0;
    std::vector<uint16_t> raw(count);
    const size_t got = count ? fread(raw.data(), sizeof(uint16_t), count, fp) : 0;
    fclose(fp);
    if (got != count || count <= 2 * size_t(seq_len)) return GPTB200_ERR_INVALID_ARG;   // not even one batch (data_loader.cpp:95)
    gptb200_loader *ld = new gptb200_loader();
    ld->seq_len = seq_len;
    ld->data.assign(raw.begin(), raw.end());
    ld->order.resize(count / seq_len - 1);   // - 1: room for the epoch's base offset
    *out = ld;
    return GPTB200_OK;
}

int gptb200_loader_destroy(gptb200_loader *ld)
{
    delete ld;
    return GPTB200_OK;
}

long long gptb200_loader_num_samples(const gptb200_loader *ld) { return ld ? static_cast<long long>(ld->order.size()) : -1; }

// Draws the epoch's base offset and shuffle from rand(), exactly as DataLoader::reset_epoch (data_loader.cpp:115-134).
int gptb200_loader_reset_epoch(gptb200_loader *ld)
{
    if (!ld) return GPTB200_ERR_INVALID_ARG;
    const size_t base = size_t(rand()) % size_t(ld->seq_len);
    const size_t n = ld->order.size();
    for (size_t i = 0; i < n; ++i) ld->order[i] = static_cast<int>(i * ld->seq_len + base);
    for (size_t i = n - 1; i > 0; --i) {
        const size_t j = size_t(rand()) % (i + 1);
        const int t = ld->order[i];
        ld->order[i] = ld->order[j];
        ld->order[j] = t;
    }
    ld->cursor = 0;
    return GPTB200_OK;
}

// Rank `rank` of `world`: its `batch` sequences of the next global batch into inputs / labels ([batch x seq_len] int32, host).
// Returns 1 when a batch was produced, 0 when the epoch has no full global batch left, < 0 on a bad argument.
int gptb200_loader_next_batch(gptb200_loader *ld, int rank, int world, int batch, int *inputs, int *labels)
{
    if (!ld || world <= 0 || rank < 0 || rank >= world || batch <= 0 || !inputs || !labels) return -GPTB200_ERR_INVALID_ARG;
    const size_t global = size_t(world) * batch;
    if (ld->cursor + global - 1 >= ld->order.size()) return 0;   // data_loader.cpp:138-141 with the global batch
    const size_t T = size_t(ld->seq_len);
    for (int i = 0; i < batch; ++i) {
        const int at = ld->order[ld->cursor + size_t(rank) * batch + i];
        memcpy(inputs + i * T, ld->data.data() + at, T * sizeof(int));
        memcpy(labels + i * T, ld->data.data() + at + 1, T * sizeof(int));
    }
    ld->cursor += global;
    return 1;
}

}  // extern "C"
