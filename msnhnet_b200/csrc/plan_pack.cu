// Weight arena staging and the pack cache file.
//
// While launches are planned, every packed tensor (conv weights, scale / bias tables, slopes) is laid out in
// pl->pack_host and launches hold tagged offsets; the offsets turn into device pointers once the arena's size is known.
// With plan_use_pack the laid-out bytes are also kept in a file next to the .msnhbin blob, and a later build of the same
// plan takes them (and the conv tile shapes) from there instead of repacking.
#include <fcntl.h>
#include <unistd.h>
#include <atomic>
#include "plan_internal.h"

using namespace msnh;

namespace msnh {

uint8_t *reserve_pack_bytes(MsnhB200Plan *pl, size_t bytes, void **dev) {
    const size_t off = pl->pack_cursor;
    pl->pack_cursor = (off + std::max<size_t>(bytes, 16) + 255) / 256 * 256;
    *dev = reinterpret_cast<void *>(kPackTag | off);
    if (pl->pack_loaded) return nullptr;         // (the bytes come from the pack file, which holds this tensor at this offset)
    if (pl->pack_host.size() < pl->pack_cursor) pl->pack_host.resize(pl->pack_cursor, 0);
    return pl->pack_host.data() + off;
}

namespace {

// ---- pack file: header, `bytes` of arena, then `picks` conv tile shapes (3 x int32 each: sub-tiles, channels, form)
//      in launch order ----
struct PackHeader { char magic[8]; uint64_t key; uint64_t tag; uint64_t bytes; uint64_t picks; uint64_t checksum; };
constexpr char kPackMagic[8] = {'M', 'S', 'N', 'H', 'P', 'K', '0', '3'};

uint64_t fnv1a(uint64_t h, const void *data, size_t n) {
    const uint8_t *p = static_cast<const uint8_t *>(data);
    for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
    return h;
}
// Checksum of the arena bytes and the stored shapes: four interleaved multiply-xor lanes over 8-byte words (a few GB/s,
// so that checking a 130 MB pack costs less than reading it), folded with the tail bytes.
uint64_t checksum64(const uint8_t *p, size_t n, uint64_t seed) {
    uint64_t h[4] = {seed ^ 0x9e3779b97f4a7c15ull, seed ^ 0xc2b2ae3d27d4eb4full, seed ^ 0x165667b19e3779f9ull, seed ^ 0x27d4eb2f165667c5ull};
    size_t i = 0;
    for (; i + 32 <= n; i += 32) {
        uint64_t w[4];
        std::memcpy(w, p + i, 32);
        for (int k = 0; k < 4; ++k) { h[k] = (h[k] ^ w[k]) * 0x100000001b3ull; h[k] ^= h[k] >> 29; }
    }
    uint64_t r = fnv1a(1469598103934665603ull, p + i, n - i);
    for (int k = 0; k < 4; ++k) r = (r ^ h[k]) * 0x100000001b3ull;
    return r ^ (r >> 32);
}
// Everything the arena's layout and contents depend on besides the weight values themselves.
uint64_t pack_key(const MsnhB200Plan *pl) {
    uint64_t h = 1469598103934665603ull;
    for (const OpState &o : pl->ops) h = fnv1a(h, &o.d, sizeof(o.d));
    const int32_t v[9] = {pl->in_c, pl->in_h, pl->in_w, pl->batch, pl->dtype, static_cast<int32_t>(pl->flags & (MSNH_PLAN_NO_FUSION | MSNH_PLAN_NO_TENSOR_CORE | MSNH_PLAN_KEEP_ALL)), 7 /* layout version */,
                          pl->ctx->sm_count /* the stored tile shapes were timed on this many SMs */, pl->dbg.no_merge ? 1 : 0};
    return fnv1a(h, v, sizeof(v));
}

}  // namespace

bool pack_probe(MsnhB200Plan *pl) {
    if (pl->pack_path.empty()) return false;
    const uint64_t key = pack_key(pl);
    if (pl->pack_blob_key == key && pl->pack_blob_tag == pl->pack_tag && !pl->pack_blob.empty()) return true;   // probed already (plan_use_pack)
    pl->pack_blob.clear(); pl->pack_blob_key = 0; pl->pack_picks.clear();
    FILE *f = std::fopen(pl->pack_path.c_str(), "rb");
    if (!f) return false;
    PackHeader hd{};
    bool ok = std::fread(&hd, sizeof(hd), 1, f) == 1 && std::memcmp(hd.magic, kPackMagic, 8) == 0 && hd.key == key && hd.tag == pl->pack_tag;
    // a file cut short (a writer that died, a full disk) is no pack
    ok = ok && std::fseek(f, 0, SEEK_END) == 0 && static_cast<uint64_t>(std::ftell(f)) == sizeof(hd) + hd.bytes + hd.picks * 12 &&
         std::fseek(f, sizeof(hd), SEEK_SET) == 0;
    std::vector<uint8_t> blob;
    std::vector<std::array<int32_t, 3>> picks;
    if (ok) {
        blob.resize(std::max<size_t>(hd.bytes, 1));
        picks.assign(static_cast<size_t>(hd.picks), std::array<int32_t, 3>{0, 0, 0});
        ok = std::fread(blob.data(), 1, hd.bytes, f) == hd.bytes && (hd.picks == 0 || std::fread(picks.data(), 12, picks.size(), f) == picks.size());
    }
    std::fclose(f);
    // a file whose bytes are not the ones its writer summed (a torn or damaged copy) is no pack either
    ok = ok && checksum64(reinterpret_cast<const uint8_t *>(picks.data()), picks.size() * 12, checksum64(blob.data(), hd.bytes, 0)) == hd.checksum;
    if (!ok) return false;
    pl->pack_blob.swap(blob); pl->pack_blob_bytes = hd.bytes; pl->pack_picks.swap(picks);
    pl->pack_blob_key = key; pl->pack_blob_tag = pl->pack_tag;
    return true;
}

int pack_load_arena(MsnhB200Plan *pl) {
    MsnhB200Ctx *ctx = pl->ctx;
    if (pl->pack_blob_bytes != pl->pack_cursor)
        return fail(ctx, MSNH_B200_ERR_STATE, "pack file %s holds %llu bytes, this plan lays out %zu", pl->pack_path.c_str(),
                    static_cast<unsigned long long>(pl->pack_blob_bytes), pl->pack_cursor);
    CUDA_TRY(ctx, cudaMemcpy(pl->d_pack, pl->pack_blob.data(), pl->pack_cursor, cudaMemcpyHostToDevice));
    std::vector<uint8_t>().swap(pl->pack_blob);
    pl->pack_blob_key = 0;
    return MSNH_B200_OK;
}

void pack_write(MsnhB200Plan *pl) {
    // Tile shapes forced through the debug switches are not what a later, unforced build should inherit.
    if (pl->dbg.forces_tiles()) return;
    // Written under a temporary name that is this process's own (created exclusively, so that two ranks building the same
    // net never share a file) and renamed when complete, so that a reader never sees half a file.
    static std::atomic<unsigned> serial{0};
    char suffix[64];
    snprintf(suffix, sizeof(suffix), ".tmp.%ld.%u", static_cast<long>(getpid()), serial.fetch_add(1));
    const std::string tmp = pl->pack_path + suffix;
    PackHeader hd{};
    std::memcpy(hd.magic, kPackMagic, 8); hd.key = pack_key(pl); hd.tag = pl->pack_tag; hd.bytes = pl->pack_cursor; hd.picks = pl->pack_picks.size();
    hd.checksum = checksum64(reinterpret_cast<const uint8_t *>(pl->pack_picks.data()), pl->pack_picks.size() * 12, checksum64(pl->pack_host.data(), pl->pack_cursor, 0));
    const int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_EXCL, 0644);
    FILE *f = fd >= 0 ? fdopen(fd, "wb") : nullptr;
    if (!f && fd >= 0) ::close(fd);
    bool ok = f && std::fwrite(&hd, sizeof(hd), 1, f) == 1 && std::fwrite(pl->pack_host.data(), 1, pl->pack_cursor, f) == pl->pack_cursor &&
              (pl->pack_picks.empty() || std::fwrite(pl->pack_picks.data(), 12, pl->pack_picks.size(), f) == pl->pack_picks.size());
    if (f) ok = (std::fclose(f) == 0) && ok;
    if (!ok || std::rename(tmp.c_str(), pl->pack_path.c_str()) != 0) { if (fd >= 0) std::remove(tmp.c_str()); }   // the cache is best effort
}

}  // namespace msnh
