// Host side of the byte-activation binary convolution (bconv_u8.cuh): geometry, tensor maps, launches, C ABI.
#include <algorithm>

#include "bconv_halo.cuh"
#include "kernels.h"

namespace dabnn {

namespace {

struct U8Plan {
    int OH = 0, OW = 0, rows = 0, imgs = 0, tiles_per_img = 0, ntiles = 0, G = 0, stages = 0, wb = 0, nboxes = 0;
    int smem = 0, resident = 0, stiles = 2, wide = 0, pair = 0, nbc = TC5_MAX_N, lag = 0;
};

// Shapes the engine takes: whole 64-channel groups, channel counts in 16s, stride 1 or 2 (even H and W), no
// dilation, output rows of at most 128 pixels.
// force_pair: -1 = pair the pixel tiles where the tile count makes it pay, 0 / 1 = the plan without / with pairing
// (the choice depends on the batch; a Net decides once whether a layer runs here, for every batch up to its maximum).
bool u8_plan(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w,
             U8Plan& pl, int force_pair = -1) {
    if (n <= 0 || h <= 0 || w <= 0 || cin <= 0 || cout <= 0 || kh <= 0 || kw <= 0 || pad_h < 0 || pad_w < 0) return false;
    if (cin % 64 || cout % 16 || stride_h != stride_w || (stride_h != 1 && stride_h != 2)) return false;
    if (stride_h == 2 && ((h | w) & 1)) return false;
    pl.OH = conv_out_dim(h, pad_h, 1, kh, stride_h);
    pl.OW = conv_out_dim(w, pad_w, 1, kw, stride_w);
    if (pl.OH <= 0 || pl.OW <= 0 || pl.OW > 128) return false;
    if ((long long)n * pl.OH * pl.OW >= (1ll << 31) || kh > 255 || kw > 255) return false;
    const int ohw = pl.OH * pl.OW;
    if (ohw <= 128) {
        pl.imgs = 128 / ohw; pl.rows = pl.OH; pl.tiles_per_img = 1;
        pl.ntiles = (n + pl.imgs - 1) / pl.imgs;
    } else {
        const int rmax = 128 / pl.OW;
        pl.tiles_per_img = (pl.OH + rmax - 1) / rmax;
        pl.rows = (pl.OH + pl.tiles_per_img - 1) / pl.tiles_per_img;
        pl.imgs = 1;
        pl.ntiles = n * pl.tiles_per_img;
    }
    pl.nboxes = kh * kw * (cin / 64);
    pl.wb = u8_weight_rows(cout);
    pl.G = pl.nboxes % 3 == 0 ? 3 : pl.nboxes % 4 == 0 ? 4 : pl.nboxes % 2 == 0 ? 2 : std::min(pl.nboxes, 3);
    // 128 input channels: one load per tap with rows of 128 bytes, a stage is one tap (a pair of boxes).  With more
    // channels the stage size decides (the kernel is bound by the bytes an SM can take in plus a fixed cost per
    // stage), and three 64-byte boxes per stage measured faster than two pairs.
    pl.wide = cin == 128;
    if (pl.wide) pl.G = 2;
    const int res_bytes = pl.nboxes * pl.wb * 64;
    pl.resident = res_bytes <= 48 * 1024;   // a channel block's weights stay in shared memory
    // with resident weights the ring carries pixel boxes only and there is room for a third staging tile
    pl.stiles = pl.resident ? 4 : 3;   // one more than the look-ahead needs: the latest tensor store may still be reading its tile
    pl.lag = 1;
    const int stile_bytes = u8_staging_tile_bytes(pl.rows * pl.OW * pl.imgs);
    int avail = U8_MAX_SMEM - 1024 - pl.stiles * stile_bytes - 3072 /* static shared memory */;
    if (pl.resident) avail -= res_bytes;
    // Streamed weights: two pixel tiles per weight stage (a stage is then two boxes of each tile and of the weights),
    // where handing out tiles in pairs does not lengthen the longest CTA's share (a few per cent per tile; a whole
    // extra tile would cost more).
    {
        const int ctas = std::max(1, sm_count() / ((cout + TC5_MAX_N - 1) / TC5_MAX_N));
        const int units = (pl.ntiles + 1) / 2;
        const bool can_pair = !pl.resident && pl.nboxes % 2 == 0;
        pl.pair = can_pair && 2 * ((units + ctas - 1) / ctas) <= (pl.ntiles + ctas - 1) / ctas;
        if (force_pair >= 0) pl.pair = can_pair && force_pair;
    }
    if (pl.pair) pl.G = 2;
    // Too few tiles for the SMs (a handful of images): narrower channel blocks, so that more CTAs share the weight stream.
    pl.nbc = TC5_MAX_N;
    if (!pl.resident && !pl.pair)
        while (pl.nbc > 32 && cout > pl.nbc / 2 && 2 * pl.ntiles * ((cout + pl.nbc - 1) / pl.nbc) <= sm_count()) pl.nbc >>= 1;
    const int stage_bytes = pl.G * ((pl.pair ? 2 : 1) * U8_BOX_BYTES + (pl.resident ? 0 : pl.wb * 64));
    pl.stages = std::min(8, avail / stage_bytes);
    if (pl.stages < 2) return false;
    pl.smem = (pl.resident ? res_bytes : 0) + pl.stages * stage_bytes + pl.stiles * stile_bytes + 1024;
    return true;
}

// maps[0] / maps[1]: the input seen from even / odd rows (the same map twice for stride 1)
bool u8_input_maps(const unsigned char* in, int n, int h, int w, int cin, int stride, const U8Plan& pl, CUtensorMap* maps) {
    const unsigned long long C = cin;
    const unsigned box[5] = {pl.wide ? 128u : 64u, (unsigned)pl.OW, (unsigned)pl.rows, (unsigned)pl.imgs, 1u};
    if (stride == 1) {
        const unsigned long long dims[5] = {C, (unsigned long long)w, (unsigned long long)h, (unsigned long long)n, 1ull};
        const unsigned long long strides[4] = {C, C * w, C * w * h, C * w * h * n};
        if (!make_u8_tensor_map(&maps[0], in, 5, dims, strides, box)) return false;
        maps[1] = maps[0];
        return true;
    }
    for (int hp = 0; hp < 2; hp++) {
        const unsigned long long dims[5] = {C, (unsigned long long)(w / 2), (unsigned long long)(h / 2), (unsigned long long)n, 2ull};
        const unsigned long long strides[4] = {2 * C, 2 * C * w, C * w * h, C};
        if (!make_u8_tensor_map(&maps[hp], in + (size_t)hp * w * cin, 5, dims, strides, box)) return false;
    }
    return true;
}

// ---- the halo kernel (bconv_halo.cuh): 3x3, stride 1, padding 1 --------------------------------------------------
struct HaloPlan {
    int OH = 0, OW = 0, P = 0, rows = 0, tiles_per_img = 0, ntiles = 0, hslots = 0, halo_stride = 0, wstages = 0, wb = 0;
    int resident = 0, stiles = 2, pair = 0, smem = 0;
    int lag = 0;                   // see HaloParams
    int imgs = 1, img_pitch = 0;   // two whole images per tile (small images): accumulator rows between them
    int nb = TC5_MAX_N;            // output channels per CTA
};

int g_halo_mode = 1;   // 0: never, 1: wherever the shape allows (dabnn_debug_set_halo)
int g_halo_stiles = 0; // 0: the plan's choice, else the number of staging tiles to try (dabnn_debug_set_halo, bits 4..7)

// even_rows: tiles of an even number of output rows (the block also writes its 2x2 average pooling)
bool halo_plan(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w,
               HaloPlan& pl, int force_pair = -1, bool even_rows = false) {
    if (!g_halo_mode || kh != 3 || kw != 3 || pad_h != 1 || pad_w != 1 || stride_h != 1 || stride_w != 1) return false;
    if (n <= 0 || h <= 0 || w <= 0 || cin % 64 || cout % 16 || cin <= 0 || cout <= 0 || w + 2 > 128) return false;
    if ((long long)n * h * w >= (1ll << 31)) return false;
    pl.OH = h; pl.OW = w; pl.P = w + 2;
    pl.imgs = 1; pl.img_pitch = 0;
    // Two whole images per tile when both fit the MMA's 128 rows at a pitch of OW + 1 (7x7: 64 + 56 rows) and the second
    // halo starts on a swizzle-atom boundary (eight pixels).
    const bool two = !even_rows && (2 * h + 1) * (w + 1) <= 128 && ((h + 1) * (w + 1)) % 8 == 0;
    if (two) {
        pl.P = w + 1;
        pl.imgs = 2; pl.img_pitch = (h + 1) * pl.P;
        pl.tiles_per_img = 1;
        pl.rows = h;
        pl.ntiles = (n + 1) / 2;
    } else {
        int rmax = 128 / pl.P;
        if (even_rows) {
            rmax &= ~1;
            if (rmax < 2 || (h & 1) || (w & 1) || (rmax / 2) * (w / 2) * 16 > U8_EPILOGUE) return false;
        }
        pl.tiles_per_img = (h + rmax - 1) / rmax;
        pl.rows = (h + pl.tiles_per_img - 1) / pl.tiles_per_img;
        if (even_rows) pl.rows = (pl.rows + 1) & ~1;   // still at most rmax, and every tile starts on an even row
        pl.ntiles = n * pl.tiles_per_img;
        // an image smaller than half a tile that cannot share it with a second one is better served by the per-tap kernel
        if (pl.rows * pl.P < 96) return false;
    }
    const int cw = cin / 64;
    pl.wb = u8_weight_rows(cout);
    const int wbox = pl.wb * 64, res_bytes = 9 * cw * wbox;
    pl.resident = res_bytes <= 48 * 1024;
    // One staging tile more than the shortcut's look-ahead needs, so that the tensor store of the block just finished may
    // still be reading its tile when the next shortcut is fetched (measured: 56x56 390 -> 374 us, 28x28 226 -> 216 us at
    // batch 1024; a deeper look-ahead bought nothing).
    pl.stiles = pl.resident ? 4 : 3;
    pl.lag = 1;
    if (g_halo_stiles) { pl.stiles = std::min(g_halo_stiles & 7, U8_MAX_STILES); pl.lag = (g_halo_stiles >> 3) & 1; }
    pl.halo_stride = (((pl.img_pitch + (pl.rows + 2) * pl.P + (two ? 1 : 0)) * 64) + 1023) & ~1023;
    const int stile_bytes = u8_staging_tile_bytes(pl.imgs * pl.rows * pl.OW);
    int avail = U8_MAX_SMEM - 1024 - pl.stiles * stile_bytes - 3072 /* static shared memory */;
    {
        const int ctas = std::max(1, sm_count() / ((cout + TC5_MAX_N - 1) / TC5_MAX_N));
        const int units = (pl.ntiles + 1) / 2;
        pl.pair = !pl.resident && 2 * ((units + ctas - 1) / ctas) <= (pl.ntiles + ctas - 1) / ctas;
        if (force_pair >= 0) pl.pair = !pl.resident && force_pair;
    }
    const int np = pl.pair ? 2 : 1;
    // Too few tiles for the SMs (a handful of images): narrower channel blocks, so that more CTAs share the weight stream.
    pl.nb = TC5_MAX_N;
    if (!pl.resident && !pl.pair)
        while (pl.nb > 32 && cout > pl.nb / 2 && 2 * pl.ntiles * ((cout + pl.nb - 1) / pl.nb) <= sm_count()) pl.nb >>= 1;
    const int wboxs = std::min(pl.nb, pl.wb) * 64;   // this CTA's rows of a box image
    if (pl.resident) {
        avail -= res_bytes;
        pl.wstages = 0;
    } else {
        // weight ring first (two to four stages of three boxes), the halo ring gets the rest
        pl.wstages = 0;
        // (narrow channel blocks: small stages, and the launch is a race against L2 latency - keep more of them in flight)
        for (int ws = pl.nb < TC5_MAX_N ? HL_MAX_WSTAGES : 4; ws >= 2 && !pl.wstages; ws--)
            if ((avail - ws * 3 * wboxs) / pl.halo_stride >= std::min(HL_MAX_HSLOTS, 2 * np * std::min(cw, 2))) pl.wstages = ws;
        if (!pl.wstages) pl.wstages = 2;
        avail -= pl.wstages * 3 * wboxs;
    }
    pl.hslots = std::min(HL_MAX_HSLOTS, avail / pl.halo_stride);
    if (pl.hslots < 2 * np) return false;
    pl.smem = 1024 + pl.hslots * pl.halo_stride + (pl.resident ? res_bytes : pl.wstages * 3 * wboxs) + pl.stiles * stile_bytes;
    return true;
}

bool halo_input_map(const unsigned char* in, int n, int h, int w, int cin, const HaloPlan& pl, CUtensorMap* map) {
    const unsigned long long C = cin;
    const unsigned box[5] = {64u, (unsigned)pl.P, (unsigned)(pl.rows + 2), 1u, 1u};
    const unsigned long long dims[5] = {C, (unsigned long long)w, (unsigned long long)h, (unsigned long long)n, 1ull};
    const unsigned long long strides[4] = {C, C * w, C * w * h, C * w * h * n};
    return make_u8_tensor_map(map, in, 5, dims, strides, box);
}

}  // namespace

bool bconv_u8_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w) {
    // Both tilings must fit: which one a launch uses depends on its batch, and a Net that keeps a blob as bytes has
    // no other engine to fall back to for a smaller batch or a ragged last sub-batch.
    U8Plan pl, other;
    if (!u8_plan(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, pl, 0)) return false;
    if (!u8_plan(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, other, 1)) return false;
    // the encoder only looks at the address's alignment: try the descriptors of this shape once
    CUtensorMap maps[2];
    return u8_input_maps(reinterpret_cast<const unsigned char*>(uintptr_t(1) << 20), n, h, w, cin, stride_h, pl, maps);
}

size_t bconv_u8_weight_bytes(int cout, int nboxes) { return u8_weight_bytes(cout, nboxes); }

int bconv_u8_expand_weights(const uint64_t* weight, size_t weight_words, int cout, int nboxes, unsigned char* dst,
                            cudaStream_t stream) {
    DABNN_REQUIRE(weight && dst && cout > 0 && nboxes > 0, DABNN_ERR_ARG, "bconv_u8_expand_weights: bad arguments");
    DABNN_REQUIRE(weight_words % (size_t)cout == 0 && weight_words / cout >= (size_t)nboxes, DABNN_ERR_SHAPE,
                  "bconv_u8_expand_weights: filter rows shorter than kh*kw*cin/64 words");
    DABNN_REQUIRE((reinterpret_cast<uintptr_t>(dst) & 15) == 0, DABNN_ERR_ARG, "bconv_u8_expand_weights: dst must be 16-byte aligned");
    dim3 grid(nboxes, (cout + TC5_MAX_N - 1) / TC5_MAX_N);
    bconv_u8_expand_weights_kernel<<<grid, 256, 0, stream>>>(weight, (long long)(weight_words / cout), cout, nboxes, dst);
    return check_launch("bconv_u8_expand_weights_kernel");
}

int binarize_u8_impl(const float* in, unsigned char* out, size_t count, cudaStream_t stream) {
    if (count == 0) return DABNN_OK;
    DABNN_REQUIRE(in && out, DABNN_ERR_ARG, "binarize_u8: null pointer");
    DABNN_REQUIRE(((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0, DABNN_ERR_ARG,
                  "binarize_u8: pointers must be 16-byte aligned");
    const size_t n16 = count / 16;
    const int blocks = (int)std::min<size_t>((n16 + 255) / 256 + 1, (size_t)sm_count() * 16);
    binarize_u8_kernel<<<blocks, 256, 0, stream>>>(in, out, n16, count);
    return check_launch("binarize_u8_kernel");
}

bool bconv_u8_pool_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w) {
    HaloPlan a, b;
    return halo_plan(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, a, 0, true) &&
           halo_plan(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, b, 1, true);
}

int bconv_u8_block_impl(const unsigned char* in_u8, const unsigned char* w_img, const float* a, const float* b,
                        const float* shortcut, float* out_f32, unsigned char* out_u8, uint64_t* out_bits, int n, int h, int w,
                        int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w,
                        cudaStream_t stream, float* pool_out) {
    DABNN_REQUIRE(in_u8 && w_img, DABNN_ERR_ARG, "bconv_u8: null pointer");
    DABNN_REQUIRE((a == nullptr) == (b == nullptr), DABNN_ERR_ARG, "bconv_u8: a and b go together");
    DABNN_REQUIRE(out_f32 || out_u8 || out_bits, DABNN_ERR_ARG, "bconv_u8: no output requested");
    U8Plan pl;
    DABNN_REQUIRE(u8_plan(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, pl), DABNN_ERR_SHAPE,
                  "bconv_u8: shape not supported by the byte-activation engine");
    DABNN_REQUIRE(!out_bits || cout % 64 == 0, DABNN_ERR_SHAPE, "bconv_u8: bit output needs cout % 64 == 0");
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    DABNN_REQUIRE(al16(in_u8) && al16(w_img) && al16(shortcut) && al16(out_f32) && al16(out_u8) && al16(out_bits), DABNN_ERR_ARG,
                  "bconv_u8: pointers must be 16-byte aligned");
    static thread_local int configured_device = -1;
    int dev = 0;
    DABNN_CUDA_OK(cudaGetDevice(&dev));
    if (configured_device != dev) {
        DABNN_CUDA_OK(cudaFuncSetAttribute(bconv_u8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, U8_MAX_SMEM - 3072));
        DABNN_CUDA_OK(cudaFuncSetAttribute(bconv_u8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, U8_MAX_SMEM - 3072));
        DABNN_CUDA_OK(cudaFuncSetAttribute(bconv_halo_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, U8_MAX_SMEM - 3072));
        DABNN_CUDA_OK(cudaFuncSetAttribute(bconv_halo_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, U8_MAX_SMEM - 3072));
        configured_device = dev;
    }
    HaloPlan hp;
    DABNN_REQUIRE(!pool_out || (al16(pool_out) && halo_plan(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, hp, -1, true)), DABNN_ERR_SHAPE,
                  "bconv_u8: the pooled output needs a 3x3 stride-1 block with even height and width that the halo kernel takes");
    if (halo_plan(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w, hp, -1, pool_out != nullptr)) {   // 3x3 stride 1: every input byte enters the SM once per tile
        CUtensorMap in_map, out_map{}, sc_map{};
        DABNN_REQUIRE(halo_input_map(in_u8, n, h, w, cin, hp, &in_map), DABNN_ERR_CUDA, "bconv_u8: cannot encode the halo's tensor map");
        {
            const unsigned long long dims[3] = {(unsigned long long)cout, (unsigned long long)hp.OH * hp.OW, (unsigned long long)n};
            const unsigned long long strides[2] = {(unsigned long long)cout * 4, (unsigned long long)cout * 4 * hp.OH * hp.OW};
            const unsigned box[3] = {32u, (unsigned)(hp.rows * hp.OW), (unsigned)hp.imgs};
            DABNN_REQUIRE(!out_f32 || make_f32_tensor_map(&out_map, out_f32, 3, dims, strides, box), DABNN_ERR_CUDA,
                          "bconv_u8: cannot encode the output's tensor map");
            DABNN_REQUIRE(!shortcut || make_f32_tensor_map(&sc_map, const_cast<float*>(shortcut), 3, dims, strides, box), DABNN_ERR_CUDA,
                          "bconv_u8: cannot encode the shortcut's tensor map");
        }
        HaloParams q{};
        q.w_img = w_img; q.a = a; q.b = b; q.shortcut = shortcut; q.out = out_f32; q.out_u8 = out_u8; q.out_bits = out_bits;
        q.pool_out = pool_out;
        q.B = n; q.OH = hp.OH; q.OW = hp.OW; q.N = cout; q.cw = cin / 64; q.P = hp.P; q.imgs = hp.imgs; q.img_pitch = hp.img_pitch; q.nb = hp.nb;
        q.rows = hp.rows; q.tiles_per_img = hp.tiles_per_img; q.ntiles = hp.ntiles;
        q.hslots = hp.hslots; q.halo_stride = hp.halo_stride; q.wstages = hp.wstages; q.wb = hp.wb;
        q.resident = hp.resident; q.stiles = hp.stiles; q.pair = hp.pair; q.lag = hp.lag;
        const int tiles_n = (cout + hp.nb - 1) / hp.nb;
        const int per_n = std::max(1, sm_count() / tiles_n);
        const int nunits = hp.pair ? (hp.ntiles + 1) / 2 : hp.ntiles;
        dim3 grid(std::min(nunits, per_n), tiles_n);
        if (hp.pair) launch_overlapped(bconv_halo_kernel<true>, grid, HL_THREADS, hp.smem, stream, q, in_map, out_map, sc_map);
        else launch_overlapped(bconv_halo_kernel<false>, grid, HL_THREADS, hp.smem, stream, q, in_map, out_map, sc_map);
        return check_launch("bconv_halo_kernel");
    }
    CUtensorMap in_maps[2], out_map{}, sc_map{};
    DABNN_REQUIRE(u8_input_maps(in_u8, n, h, w, cin, stride_h, pl, in_maps), DABNN_ERR_CUDA, "bconv_u8: cannot encode the input's tensor map");
    {
        const unsigned long long dims[3] = {(unsigned long long)cout, (unsigned long long)pl.OH * pl.OW, (unsigned long long)n};
        const unsigned long long strides[2] = {(unsigned long long)cout * 4, (unsigned long long)cout * 4 * pl.OH * pl.OW};
        const unsigned box[3] = {32u, (unsigned)(pl.rows * pl.OW), (unsigned)pl.imgs};
        DABNN_REQUIRE(!out_f32 || make_f32_tensor_map(&out_map, out_f32, 3, dims, strides, box), DABNN_ERR_CUDA,
                      "bconv_u8: cannot encode the output's tensor map");
        DABNN_REQUIRE(!shortcut || make_f32_tensor_map(&sc_map, const_cast<float*>(shortcut), 3, dims, strides, box), DABNN_ERR_CUDA,
                      "bconv_u8: cannot encode the shortcut's tensor map");
    }
    U8Params p{};
    p.w_img = w_img; p.a = a; p.b = b; p.shortcut = shortcut; p.out = out_f32; p.out_u8 = out_u8; p.out_bits = out_bits;
    p.B = n; p.OH = pl.OH; p.OW = pl.OW; p.N = cout;
    p.kh = kh; p.kw = kw; p.pad_h = pad_h; p.pad_w = pad_w; p.stride = stride_h; p.cw = cin / 64;
    p.rows = pl.rows; p.imgs = pl.imgs; p.tiles_per_img = pl.tiles_per_img; p.ntiles = pl.ntiles;
    p.G = pl.G; p.stages = pl.stages; p.wb = pl.wb; p.nboxes = pl.nboxes; p.resident = pl.resident; p.stiles = pl.stiles; p.wide = pl.wide; p.pair = pl.pair; p.nbc = pl.nbc; p.lag = pl.lag;
    const int tiles_n = (cout + pl.nbc - 1) / pl.nbc;
    const int per_n = std::max(1, sm_count() / tiles_n);
    const int nunits = pl.pair ? (pl.ntiles + 1) / 2 : pl.ntiles;
    dim3 grid(std::min(nunits, per_n), tiles_n);
    if (pl.pair) launch_overlapped(bconv_u8_kernel<true>, grid, U8_THREADS, pl.smem, stream, p, in_maps[0], in_maps[1], out_map, sc_map);
    else launch_overlapped(bconv_u8_kernel<false>, grid, U8_THREADS, pl.smem, stream, p, in_maps[0], in_maps[1], out_map, sc_map);
    return check_launch("bconv_u8_kernel");
}

int bconv_u8_status_word(int** addr) {
    DABNN_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(addr), g_u8_status));
    return DABNN_OK;
}

int bconv_u8_status(int* status) {
    DABNN_CUDA_OK(cudaMemcpyFromSymbol(status, g_u8_status, sizeof(int)));
    return DABNN_OK;
}

}  // namespace dabnn

using namespace dabnn;

extern "C" int dabnn_debug_set_halo(int mode) {
    g_halo_mode = (mode & 15) != 0;
    g_halo_stiles = (mode >> 4) & 15;
    return DABNN_OK;
}

extern "C" int dabnn_binarize_u8(const float* in, unsigned char* out, size_t count, dabnn_stream_t s) {
    return binarize_u8_impl(in, out, count, static_cast<cudaStream_t>(s));
}

extern "C" int dabnn_bconv_u8_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w,
                                        int stride_h, int stride_w) {
    return bconv_u8_supported(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w) ? 1 : 0;
}

extern "C" size_t dabnn_bconv_u8_weight_bytes(int cout, int kwords) {
    return cout > 0 && kwords > 0 ? bconv_u8_weight_bytes(cout, kwords) : 0;
}

extern "C" int dabnn_bconv_u8_expand_weights(const uint64_t* weight, size_t weight_words, int cout, int kwords,
                                             unsigned char* dst, dabnn_stream_t s) {
    return bconv_u8_expand_weights(weight, weight_words, cout, kwords, dst, static_cast<cudaStream_t>(s));
}

extern "C" int dabnn_bconv_u8_block_pooled_supported(int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w,
                                                     int stride_h, int stride_w) {
    return bconv_u8_pool_supported(n, h, w, cin, cout, kh, kw, pad_h, pad_w, stride_h, stride_w) ? 1 : 0;
}

extern "C" int dabnn_bconv_u8_block_pooled(const unsigned char* in_u8, const unsigned char* w_expanded, const float* a, const float* b,
                                           const float* shortcut, float* out_f32, unsigned char* out_u8, uint64_t* out_bits, float* pool_out,
                                           int n, int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                                           int stride_w, dabnn_stream_t s) {
    DABNN_REQUIRE(pool_out, DABNN_ERR_ARG, "bconv_u8_block_pooled: null pooled output");
    return bconv_u8_block_impl(in_u8, w_expanded, a, b, shortcut, out_f32, out_u8, out_bits, n, h, w, cin, cout, kh, kw, pad_h,
                               pad_w, stride_h, stride_w, static_cast<cudaStream_t>(s), pool_out);
}

extern "C" int dabnn_bconv_u8_block(const unsigned char* in_u8, const unsigned char* w_expanded, const float* a, const float* b,
                                    const float* shortcut, float* out_f32, unsigned char* out_u8, uint64_t* out_bits, int n,
                                    int h, int w, int cin, int cout, int kh, int kw, int pad_h, int pad_w, int stride_h,
                                    int stride_w, dabnn_stream_t s) {
    return bconv_u8_block_impl(in_u8, w_expanded, a, b, shortcut, out_f32, out_u8, out_bits, n, h, w, cin, cout, kh, kw, pad_h,
                               pad_w, stride_h, stride_w, static_cast<cudaStream_t>(s));
}
