// C ABI of libtrips_b200: context (scratch owner), forward, backward, fused Adam and the inspection calls.
// The host logic here replaces PointRendererCache (src/lib/rendering/PointRenderer.cu:197-528) and the host
// parts of RenderFast16 / BlendBackwardsBilinearFast / MyAdam::step.
#include <algorithm>
#include <cfloat>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

using namespace trips;

namespace
{
struct DevBuf
{
    void* p      = nullptr;
    size_t bytes = 0;
};

inline cudaError_t ensure(DevBuf& b, size_t bytes, double growth = 1.0)
{
    if (bytes <= b.bytes) return cudaSuccess;
    if (b.p) cudaFree(b.p);
    b.p          = nullptr;
    b.bytes      = 0;
    size_t want  = (size_t)((double)bytes * growth);
    want         = (want + 255) & ~(size_t)255;
    cudaError_t e = cudaMalloc(&b.p, want);
    if (e != cudaSuccess && want > bytes)
    {
        (void)cudaGetLastError();
        want = (bytes + 255) & ~(size_t)255;
        e    = cudaMalloc(&b.p, want);
    }
    if (e == cudaSuccess) b.bytes = want;
    return e;
}
// Optional CUDA-event timers around every stage (the reference's SAIGA_OPTIONAL_TIME_MEASURE scopes,
// RenderForward.cu:1090,1166,1238,1271, PointRenderer.cu:1338) and a launch counter per stage.
struct StageTimers
{
    bool enabled = false;
    struct Span
    {
        int stage;
        cudaEvent_t a, b;
    };
    std::vector<Span> open;                            // recorded, not yet read back
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pool;  // reusable event pairs
    double ms[TRIPS_NUM_STAGES]        = {};
    int64_t launches[TRIPS_NUM_STAGES] = {};
    int64_t timed[TRIPS_NUM_STAGES]    = {};

    bool begin(int stage, cudaStream_t st, Span& sp)
    {
        if (!enabled) return false;
        if (pool.empty())
        {
            cudaEvent_t a, b;
            if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return false;
            pool.emplace_back(a, b);
        }
        sp.stage = stage;
        sp.a     = pool.back().first;
        sp.b     = pool.back().second;
        pool.pop_back();
        cudaEventRecord(sp.a, st);
        return true;
    }
    void end(const Span& sp, cudaStream_t st)
    {
        cudaEventRecord(sp.b, st);
        open.push_back(sp);
    }
    void collect()
    {
        for (const Span& sp : open)
        {
            float t = 0.f;
            if (cudaEventSynchronize(sp.b) == cudaSuccess && cudaEventElapsedTime(&t, sp.a, sp.b) == cudaSuccess)
            {
                ms[sp.stage] += t;
                timed[sp.stage] += 1;
            }
            pool.emplace_back(sp.a, sp.b);
        }
        open.clear();
    }
    void destroy()
    {
        collect();
        for (auto& pr : pool)
        {
            cudaEventDestroy(pr.first);
            cudaEventDestroy(pr.second);
        }
        pool.clear();
    }
};
}  // namespace

struct SizeKey
{
    int N, B, w, h, L, C, train;
    int layer_rule;  // which layers a point is written to (use_layer_point_size, render_points_in_all_lower_resolutions): changes the fragment count
    bool operator==(const SizeKey& o) const
    {
        return N == o.N && B == o.B && w == o.w && h == o.h && L == o.L && C == o.C && train == o.train && layer_rule == o.layer_rule;
    }
};

struct TripsContext
{
    StageTimers timers;
    int device   = 0;
    int sm_count = 148;
    std::string error;
    // forward scratch
    DevBuf heavy, views, cams, bin_count, bin_base, view_total, bin_cursor, entry_base, entries, counts, offsets, partial, view_base, frags, rec_n, records, stats, ticket, rank, rank_scratch, rank_temp, resize_scratch, block_box, block_skip;
    // backward scratch
    DevBuf egrad, g_point, g_conf_pt, g_small;
    // adam
    DevBuf adam_tab;
    // pinned host mirror of DevStats and the event behind which it becomes valid when a call did not wait for it
    void* h_pinned        = nullptr;
    cudaEvent_t totals_ev = nullptr;
    bool pending          = false;  // the totals of the last forward call have not been read yet
    // sizes the last training call needed, and the shapes they belong to
    SizeKey size_key{};
    bool have_sizes                 = false;
    unsigned long long need_entries = 0, need_frags = 0;
    int entry_C                     = 0;  // channel count the entry arrays are laid out for
    bool crowded                    = false;  // the point cloud crowds into few screen tiles: use the aggregating binning kernels
    // state of the last forward call
    bool have_forward = false;
    Geom geom{};
    TripsRenderParams params{};
    int B = 0, N = 0, n_tex = 0, C = 0;
    int nchunks = 0;
    int rank_points = -1;                  // number of points the spatial ranks were computed for (-1: none yet)
    int rank_age    = 0;                   // training forward passes since then
    size_t entry_cap = 0;                  // entries the two entry arrays (head | tail, in this order) are laid out for
    TripsStats host_stats{};
};

#define CU_CHECK(ctx, expr)                                                                      \
    do                                                                                           \
    {                                                                                            \
        cudaError_t _e = (expr);                                                                 \
        if (_e != cudaSuccess)                                                                   \
        {                                                                                        \
            (ctx)->error = std::string(#expr) + ": " + cudaGetErrorString(_e);                   \
            (void)cudaGetLastError();                                                            \
            return _e == cudaErrorMemoryAllocation ? TRIPS_ERR_OUT_OF_MEMORY : TRIPS_ERR_CUDA;   \
        }                                                                                        \
    } while (0)

// Runs `expr` (which launches `n` kernels of `stage`) between two events when the stage timers are on.
#define STAGE(ctx, stage, n, st, expr)                      \
    do                                                      \
    {                                                       \
        StageTimers::Span _sp;                              \
        bool _t = (ctx)->timers.begin((stage), (st), _sp);  \
        cudaError_t _se = (expr);                           \
        if (_t) (ctx)->timers.end(_sp, (st));               \
        (ctx)->timers.launches[(stage)] += (n);             \
        CU_CHECK(ctx, _se);                                 \
    } while (0)

static int fail(TripsContext* ctx, int code, const char* msg)
{
    if (ctx) ctx->error = msg;
    return code;
}

static void free_buf(DevBuf& b)
{
    if (b.p) cudaFree(b.p);
    b.p     = nullptr;
    b.bytes = 0;
}

static ScenePtrs scene_ptrs(const TripsScene* s)
{
    ScenePtrs sp;
    sp.N          = s->n_points;
    sp.n_tex      = s->n_tex;
    sp.C          = s->channels;
    sp.position   = reinterpret_cast<const float4*>(s->position);
    sp.point_size = s->point_size;
    sp.index      = s->index;
    sp.texture    = s->texture;
    sp.confidence = s->confidence;
    sp.background = s->background;
    sp.dropout    = s->dropout;
    return sp;
}

static FwdBuffers fwd_buffers(TripsContext* c)
{
    FwdBuffers fb;
    fb.bin_count  = (uint32_t*)c->bin_count.p;
    fb.bin_base   = (uint32_t*)c->bin_base.p;
    fb.view_total = (uint32_t*)c->view_total.p;
    fb.bin_cursor = (uint32_t*)c->bin_cursor.p;
    fb.entry_base = (unsigned long long*)c->entry_base.p;
    fb.ent_head   = (float4*)c->entries.p;
    fb.ent_tail   = (float*)c->entries.p + 8 * c->entry_cap;
    fb.counts     = (uint32_t*)c->counts.p;
    fb.offsets    = (uint32_t*)c->offsets.p;
    fb.partial    = (uint32_t*)c->partial.p;
    fb.view_base  = (unsigned long long*)c->view_base.p;
    fb.frags      = (uint4*)c->frags.p;
    fb.frag_cap   = c->frags.bytes / sizeof(uint4);
    fb.rec_n      = (uint8_t*)c->rec_n.p;
    fb.records    = (uint2*)c->records.p;
    fb.stats      = (DevStats*)c->stats.p;
    fb.ticket     = (unsigned int*)c->ticket.p;
    fb.point_rank = c->rank_points >= 0 ? (const uint32_t*)c->rank.p : nullptr;
    fb.block_box  = (const float*)c->block_box.p;
    fb.block_skip = (const uint8_t*)c->block_skip.p;
    fb.heavy      = (uint2*)c->heavy.p;
    return fb;
}

// DevStats is allocated once and zeroed then; afterwards only its counters are cleared per call.
static cudaError_t ensure_stats(TripsContext* c, cudaStream_t st)
{
    if (c->stats.p) return cudaSuccess;
    cudaError_t e = ensure(c->stats, sizeof(DevStats));
    if (e != cudaSuccess) return e;
    return cudaMemsetAsync(c->stats.p, 0, sizeof(DevStats), st);
}

static cudaError_t clear_counters(TripsContext* c, cudaStream_t st)
{
    static_assert(offsetof(DevStats, status) + sizeof(unsigned) == offsetof(DevStats, culled_blocks), "the counters lie on either side of the status word");
    cudaError_t e = cudaMemsetAsync(c->stats.p, 0, offsetof(DevStats, status), st);
    if (e != cudaSuccess) return e;
    return cudaMemsetAsync((char*)c->stats.p + offsetof(DevStats, culled_blocks), 0, sizeof(unsigned int), st);
}

static bool valid_channels(int c) { return c == 3 || c == 4 || c == 6 || c == 8 || c == 16; }

extern "C" {

const char* trips_status_string(int status)
{
    switch (status)
    {
        case TRIPS_OK: return "ok";
        case TRIPS_ERR_INVALID_ARG: return "invalid argument";
        case TRIPS_ERR_CUDA: return "CUDA error";
        case TRIPS_ERR_OUT_OF_MEMORY: return "out of device memory";
        case TRIPS_ERR_UNSUPPORTED: return "unsupported camera model or flag";
        case TRIPS_ERR_NO_FORWARD: return "backward without a training forward pass";
        case TRIPS_ERR_TOO_LARGE: return "size beyond the supported maximum";
        default: return "unknown status";
    }
}

const char* trips_last_error(const TripsContext* ctx) { return ctx ? ctx->error.c_str() : "null context"; }

int trips_context_create(TripsContext** out, int device)
{
    if (!out) return TRIPS_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count)
    {
        (void)cudaGetLastError();
        return TRIPS_ERR_CUDA;
    }
    TripsContext* c = new (std::nothrow) TripsContext();
    if (!c) return TRIPS_ERR_OUT_OF_MEMORY;
    c->device = device;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) c->sm_count = prop.multiProcessorCount;
    *out = c;
    return TRIPS_OK;
}

void trips_context_destroy(TripsContext* c)
{
    if (!c) return;
    DevBuf* all[] = {&c->heavy, &c->views, &c->cams, &c->bin_count, &c->bin_base, &c->view_total, &c->bin_cursor, &c->entry_base, &c->entries, &c->counts, &c->offsets,
                     &c->partial, &c->view_base, &c->frags, &c->rec_n, &c->records, &c->stats, &c->ticket, &c->egrad, &c->g_point,
                     &c->g_conf_pt, &c->g_small, &c->adam_tab, &c->rank, &c->rank_scratch, &c->rank_temp, &c->resize_scratch, &c->block_box, &c->block_skip};
    for (DevBuf* b : all) free_buf(*b);
    c->timers.destroy();
    if (c->h_pinned) cudaFreeHost(c->h_pinned);
    if (c->totals_ev) cudaEventDestroy(c->totals_ev);
    delete c;
}

// Geometry of the pyramid and of the tile / bin decompositions for a (w, h, L) image.
static bool make_geom(int w, int h, int L, Geom& g)
{
    g.L = L;
    long long base = 0;
    int lw = w, lh = h;
    for (int l = 0; l < g.L; ++l)
    {
        g.W[l]    = lw;
        g.H[l]    = lh;
        g.base[l] = (int)base;
        base += (long long)lw * lh;
        lw = (lw + 1) / 2;  // ceil halving, PointRenderer.cu:385-389
        lh = (lh + 1) / 2;
    }
    for (int l = g.L; l <= TRIPS_MAX_LAYERS; ++l) g.base[l] = (int)base;
    if (base > (1ll << 30)) return false;
    g.P = (int)base;
    static const int kRegTiles[5] = {0, 128, 160, 168, 170};
    g.reg_layers = g.L < 4 ? g.L : 4;
    g.reg_x      = (w + 63) / 64;
    g.reg_tiles  = kRegTiles[g.reg_layers];
    g.reg_total  = g.reg_x * ((h + 63) / 64) * g.reg_tiles;
    int tb = g.reg_total;
    for (int l = 0; l < TRIPS_MAX_LAYERS; ++l)
    {
        g.tile_base[l] = tb;
        g.tiles_x[l]   = 1;
        if (l >= g.reg_layers && l < g.L)
        {
            g.tiles_x[l] = (g.W[l] + kTileW - 1) / kTileW;
            tb += g.tiles_x[l] * ((g.H[l] + kTileH - 1) / kTileH);
        }
    }
    g.tile_base[TRIPS_MAX_LAYERS] = tb;
    g.n_tiles = tb;
    g.bins_x  = ((w - 1) >> kBinShift) + 1;
    g.bins_y  = ((h - 1) >> kBinShift) + 1;
    g.n_bins  = g.bins_x * g.bins_y;
    return true;
}

// The entry arrays (head | tail, in this order) re-laid out for at least `entries` entries.
static cudaError_t ensure_entries(TripsContext* ctx, size_t entries, int C, double growth)
{
    const size_t ES = (size_t)entry_stride(C);
    if (ctx->entries.p && ctx->entry_C == C && entries <= ctx->entry_cap) return cudaSuccess;
    const size_t want = (size_t)((double)(entries > 0 ? entries : 1) * growth) + 1;
    cudaError_t e = ensure(ctx->entries, sizeof(float) * ES * want + 16);
    if (e != cudaSuccess)
    {
        ctx->entry_cap = 0;
        return e;
    }
    ctx->entry_cap = (ctx->entries.bytes - 16) / (sizeof(float) * ES);
    ctx->entry_C   = C;
    return cudaSuccess;
}

// Totals of a forward call whose sizes were not waited for (steady-state training): read them now, publish the
// statistics, and grow the entry / fragment buffers if that call needed more than they hold (the call itself rendered
// the views that did not fit as background and raised a status bit).
static int resolve_pending(TripsContext* ctx)
{
    if (!ctx->pending) return TRIPS_OK;
    ctx->pending = false;
    CU_CHECK(ctx, cudaEventSynchronize(ctx->totals_ev));
    const DevStats* hs = (const DevStats*)ctx->h_pinned;
    ctx->need_entries  = hs->visible;
    ctx->need_frags    = hs->frag_need;
    ctx->crowded       = hs->max_key >= kHotKey;
    ctx->host_stats.visible_points      = (int64_t)hs->visible;
    ctx->host_stats.fragments           = (int64_t)hs->frag_need;
    ctx->host_stats.kept_fragments      = (int64_t)hs->kept;
    ctx->host_stats.max_list_length     = (int64_t)hs->max_len;
    ctx->host_stats.culled_point_blocks = (int64_t)hs->culled_blocks;
    return TRIPS_OK;
}

namespace
{
constexpr double kGrowth      = 1.25;  // head room of the entry / fragment buffers over the counted need
constexpr int kEvalSubBatch   = 8;     // views rendered per pass when nothing has to be kept for a backward pass
}  // namespace

// One pass over `B` views (all views of a training call; up to kEvalSubBatch views of an inference call).
//   wait_for_sizes = true : the entry and fragment buffers are sized from this pass's own counts, which costs two host
//                           synchronisations (the reference synchronises 2 * num_layers times per view for the same
//                           purpose, RenderForward.cu:1201-1208);
//   wait_for_sizes = false: the buffers keep the capacity found by earlier calls (need x 1.25) and nothing is waited
//                           for: the totals travel to pinned host memory behind an event that the next call reads.
static int forward_views(TripsContext* ctx, const TripsScene* scene, const TripsView* views, int B, const TripsRenderParams* params,
                         const Geom& g, float* const* out_layers, size_t out_view_offset, const float* dropout, cudaStream_t st,
                         bool wait_for_sizes)
{
    const size_t N    = (size_t)scene->n_points;
    const size_t P    = (size_t)g.P;
    const int C       = scene->channels;
    const int nchunks = (int)((P + kScanChunk - 1) / kScanChunk);
    const size_t n_box = (N + 8191) / 8192 + 1;

    CU_CHECK(ctx, ensure(ctx->views, sizeof(TripsView) * B));
    CU_CHECK(ctx, ensure(ctx->cams, sizeof(CamConst) * B));
    CU_CHECK(ctx, ensure(ctx->bin_count, sizeof(uint32_t) * (size_t)g.n_bins * 32 * B));  // one counter per (bin, 8x4 tile of the bin)
    CU_CHECK(ctx, ensure(ctx->bin_base, sizeof(uint32_t) * (size_t)g.n_bins * 32 * B));
    CU_CHECK(ctx, ensure(ctx->view_total, sizeof(uint32_t) * B));
    CU_CHECK(ctx, ensure(ctx->bin_cursor, sizeof(uint32_t) * (size_t)g.n_bins * B));
    CU_CHECK(ctx, ensure(ctx->entry_base, sizeof(unsigned long long) * (B + 1)));
    CU_CHECK(ctx, ensure(ctx->block_box, sizeof(float) * 6 * n_box));
    CU_CHECK(ctx, ensure(ctx->block_skip, (size_t)B * n_box));
    CU_CHECK(ctx, ensure(ctx->heavy, sizeof(uint2) * (size_t)kHeavyCap));
    CU_CHECK(ctx, ensure(ctx->counts, sizeof(uint32_t) * P * B));
    CU_CHECK(ctx, ensure(ctx->offsets, sizeof(uint32_t) * P * B));
    CU_CHECK(ctx, ensure(ctx->partial, sizeof(uint32_t) * (size_t)nchunks * B));
    CU_CHECK(ctx, ensure(ctx->view_base, sizeof(unsigned long long) * (B + 1)));
    CU_CHECK(ctx, ensure_stats(ctx, st));
    CU_CHECK(ctx, ensure(ctx->ticket, sizeof(unsigned) * (size_t)(B > 64 ? B : 64)));
    if (params->train)
    {
        CU_CHECK(ctx, ensure(ctx->rec_n, P * B));
        CU_CHECK(ctx, ensure(ctx->records, sizeof(uint2) * 16 * P * B));
    }
    if (ctx->frags.bytes == 0) CU_CHECK(ctx, ensure(ctx->frags, 16 * 1024 * 1024));
    if (!ctx->entries.p || ctx->entry_C != C) CU_CHECK(ctx, ensure_entries(ctx, 1024, C, 1.0));
    if (!ctx->h_pinned)
    {
        CU_CHECK(ctx, cudaMallocHost(&ctx->h_pinned, sizeof(DevStats)));
        CU_CHECK(ctx, cudaEventCreateWithFlags(&ctx->totals_ev, cudaEventDisableTiming));
    }
    DevStats* h_stats = (DevStats*)ctx->h_pinned;

    ScenePtrs sp = scene_ptrs(scene);
    sp.dropout   = dropout;
    // Spatial ranks of the points (where their gradient rows live, rank.cu): training only; refreshed when the number
    // of points changes and every kRankRefresh forward passes, since points move slowly and a stale rank is still a
    // valid permutation.  Entries carry the rank, so the backward pass of this forward pass sees the same ranks.
    constexpr int kRankRefresh = 512;
    if (params->train && N > 0 && N < (size_t)kMaxRankedPoints)
    {
        if (ctx->rank_points != (int)N || ctx->rank_age >= kRankRefresh)
        {
            const size_t tb = rank_temp_bytes((int)N);
            CU_CHECK(ctx, ensure(ctx->rank, sizeof(uint32_t) * N));
            CU_CHECK(ctx, ensure(ctx->rank_scratch, sizeof(uint32_t) * (4 * N + 8)));
            CU_CHECK(ctx, ensure(ctx->rank_temp, tb));
            CU_CHECK(ctx, launch_point_rank((const float4*)scene->position, (int)N, (unsigned*)ctx->rank_scratch.p, ctx->rank_temp.p, tb,
                                            (unsigned*)ctx->rank.p, ctx->sm_count, st));
            ctx->rank_points = (int)N;
            ctx->rank_age    = 0;
        }
        ++ctx->rank_age;
    }
    else
        ctx->rank_points = -1;
    FwdBuffers fb = fwd_buffers(ctx);
    // the counters start from zero; the status word keeps the bits raised by earlier calls until trips_last_status reads them
    CU_CHECK(ctx, clear_counters(ctx, st));
    CU_CHECK(ctx, cudaMemsetAsync(ctx->counts.p, 0, sizeof(uint32_t) * P * B, st));
    // the view table comes from pageable host memory: the copy is staged before the call returns
    CU_CHECK(ctx, cudaMemcpyAsync(ctx->views.p, views, sizeof(TripsView) * B, cudaMemcpyHostToDevice, st));
    STAGE(ctx, TRIPS_STAGE_SETUP, 1, st,
          launch_setup_cams((const TripsView*)ctx->views.p, B, scene->poses, scene->n_images, scene->intrinsics,
                            scene->n_cameras, params->distortion, params->dist_cutoff, (CamConst*)ctx->cams.p, fb.stats, st));
    const CamConst* cams = (const CamConst*)ctx->cams.p;
    // crowded: the last call that reported back saw more than kHotKey visible points in one (view, bin, tile) group
    STAGE(ctx, TRIPS_STAGE_BIN_POINTS, bin_count_launches((int)N, B), st,
          launch_bin_count(sp, cams, g, *params, B, fb, wait_for_sizes ? ~0ull : (unsigned long long)ctx->entry_cap, ctx->crowded, ctx->sm_count, st));
    if (wait_for_sizes)
    {
        CU_CHECK(ctx, cudaMemcpyAsync(h_stats, ctx->stats.p, sizeof(DevStats), cudaMemcpyDeviceToHost, st));
        CU_CHECK(ctx, cudaStreamSynchronize(st));
        CU_CHECK(ctx, ensure_entries(ctx, (size_t)h_stats->visible, C, kGrowth));
        ctx->crowded = h_stats->max_key >= kHotKey;  // this call's own count pass already knows
        fb           = fwd_buffers(ctx);
    }
    STAGE(ctx, TRIPS_STAGE_BIN_POINTS, bin_scatter_launches((int)N, B), st, launch_bin_scatter(sp, cams, g, *params, B, fb, ctx->crowded, ctx->sm_count, st));
    if (N > 0) STAGE(ctx, TRIPS_STAGE_COUNT, 1, st, launch_count(sp, g, B, fb, strict_layers(*params), wait_for_sizes ? (unsigned long long)h_stats->visible : ctx->need_entries, ctx->sm_count, st));
    {
        FwdBuffers fscan = fb;
        if (wait_for_sizes) fscan.frag_cap = ~0ull;  // sizing pass: the list buffer is grown below, nothing can overflow yet
        STAGE(ctx, TRIPS_STAGE_SCAN, 3, st, launch_scan(g, B, params->k_keep, fscan, nchunks, st));
    }
    CU_CHECK(ctx, cudaMemcpyAsync(h_stats, ctx->stats.p, sizeof(DevStats), cudaMemcpyDeviceToHost, st));
    if (wait_for_sizes)
    {
        CU_CHECK(ctx, cudaStreamSynchronize(st));
        if ((size_t)h_stats->frag_need * sizeof(uint4) > ctx->frags.bytes)
        {
            CU_CHECK(ctx, ensure(ctx->frags, (size_t)h_stats->frag_need * sizeof(uint4), kGrowth));
            fb = fwd_buffers(ctx);
        }
        ctx->need_entries = h_stats->visible;
        ctx->need_frags   = h_stats->frag_need;
        ctx->host_stats.visible_points += (int64_t)h_stats->visible;
        ctx->host_stats.fragments += (int64_t)h_stats->frag_need;
        ctx->host_stats.kept_fragments += (int64_t)h_stats->kept;
        ctx->host_stats.max_list_length = std::max<int64_t>(ctx->host_stats.max_list_length, (int64_t)h_stats->max_len);
        ctx->host_stats.culled_point_blocks += (int64_t)h_stats->culled_blocks;
    }
    else
    {
        CU_CHECK(ctx, cudaEventRecord(ctx->totals_ev, st));
        ctx->pending = true;
    }
    if (N > 0) STAGE(ctx, TRIPS_STAGE_COLLECT, 1, st, launch_collect(sp, g, B, fb, strict_layers(*params), ctx->sm_count, st));
    LayerPtrs out{};
    for (int l = 0; l < g.L; ++l) out.p[l] = out_layers[l] + out_view_offset * (size_t)C * g.W[l] * g.H[l];
    if (second_pipeline(*params))
        STAGE(ctx, TRIPS_STAGE_SORT_BLEND, 1, st, launch_second_blend(sp, g, *params, B, fb, out, ctx->sm_count, st));
    else
        STAGE(ctx, TRIPS_STAGE_SORT_BLEND, 2, st, [&]() -> cudaError_t {
            cudaError_t e = launch_heavy_topk(g, B, fb, ctx->sm_count, st);
            return e != cudaSuccess ? e : launch_sort_blend(sp, g, *params, B, fb, out, ctx->sm_count, st);
        }());
    ctx->B       = B;
    ctx->nchunks = nchunks;
    return TRIPS_OK;
}

int trips_forward(TripsContext* ctx, const TripsScene* scene, const TripsView* views, int n_views,
                  const TripsRenderParams* params, float* const* out_layers, void* stream)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    if (!scene || !views || !params || !out_layers || n_views < 1) return fail(ctx, TRIPS_ERR_INVALID_ARG, "null argument");
    if (params->num_layers < 1 || params->num_layers > TRIPS_MAX_LAYERS) return fail(ctx, TRIPS_ERR_INVALID_ARG, "num_layers must be 1..8");
    if (params->k_keep < 1 || params->k_keep > TRIPS_MAX_KEEP) return fail(ctx, TRIPS_ERR_INVALID_ARG, "k_keep must be 1..16");
    if (!valid_channels(scene->channels)) return fail(ctx, TRIPS_ERR_INVALID_ARG, "channels must be 3, 4, 6, 8 or 16");
    if (scene->n_points < 0 || scene->n_tex < 1 || scene->n_images < 1 || scene->n_cameras < 1)
        return fail(ctx, TRIPS_ERR_INVALID_ARG, "bad scene sizes");
    if (scene->n_points > 0 && (!scene->position || !scene->point_size)) return fail(ctx, TRIPS_ERR_INVALID_ARG, "null point arrays");
    if (!scene->texture || !scene->confidence || !scene->background || !scene->poses || !scene->intrinsics)
        return fail(ctx, TRIPS_ERR_INVALID_ARG, "null scene arrays");
    if (!scene->index && scene->n_tex < scene->n_points) return fail(ctx, TRIPS_ERR_INVALID_ARG, "identity index needs n_tex >= n_points");
    const int w = views[0].w, h = views[0].h;
    if (w < 2 || h < 2) return fail(ctx, TRIPS_ERR_INVALID_ARG, "image must be at least 2x2");
    for (int b = 0; b < n_views; ++b)
    {
        if (views[b].w != w || views[b].h != h) return fail(ctx, TRIPS_ERR_INVALID_ARG, "all views of a call must share (w, h)");
        if (views[b].camera_model_type != 0) return fail(ctx, TRIPS_ERR_UNSUPPORTED, "only the pinhole camera model is implemented");
        if (views[b].image_index < 0 || views[b].image_index >= scene->n_images || views[b].camera_index < 0 ||
            views[b].camera_index >= scene->n_cameras)
            return fail(ctx, TRIPS_ERR_INVALID_ARG, "view index out of range");
    }
    for (int l = 0; l < params->num_layers; ++l)
        if (!out_layers[l]) return fail(ctx, TRIPS_ERR_INVALID_ARG, "null output layer");
    cudaStream_t st = (cudaStream_t)stream;
    ctx->have_forward = false;
    {
        const int rs = resolve_pending(ctx);
        if (rs != TRIPS_OK) return rs;
    }
    Geom g{};
    if (!make_geom(w, h, params->num_layers, g)) return fail(ctx, TRIPS_ERR_TOO_LARGE, "pyramid has more than 2^30 pixels");
    const int B    = n_views;
    const size_t N = (size_t)scene->n_points;
    if (N * 4ull * g.L >= (1ull << 32)) return fail(ctx, TRIPS_ERR_TOO_LARGE, "a view could hold more than 2^32 fragments");
    if ((unsigned long long)B * (unsigned long long)g.n_tiles >= (1ull << 32)) return fail(ctx, TRIPS_ERR_TOO_LARGE, "too many pixel tiles");

    const SizeKey key{scene->n_points, B, w, h, params->num_layers, scene->channels, params->train,
                      (params->use_layer_point_size ? 1 : 0) | (params->render_points_in_all_lower_resolutions ? 2 : 0)};
    ctx->host_stats        = TripsStats{};
    ctx->host_stats.pixels = (int64_t)g.P * B;
    ctx->geom              = g;
    ctx->params            = *params;
    ctx->N                 = (int)N;
    ctx->n_tex             = scene->n_tex;
    ctx->C                 = scene->channels;
    if (params->train)
    {
        // Steady state of a training loop: same shapes as the previous training call.  The buffers keep the capacity that
        // call needed (x 1.25), grown here if its totals (read above, long after they were produced) say so.
        bool steady = ctx->have_sizes && key == ctx->size_key;
        if (steady)
        {
            if (ctx->need_entries > ctx->entry_cap)
                steady = ensure_entries(ctx, (size_t)ctx->need_entries, scene->channels, kGrowth) == cudaSuccess;
            if (steady && (size_t)ctx->need_frags * sizeof(uint4) > ctx->frags.bytes)
                steady = ensure(ctx->frags, (size_t)ctx->need_frags * sizeof(uint4), kGrowth) == cudaSuccess;
            (void)cudaGetLastError();
        }
        const int rc = forward_views(ctx, scene, views, B, params, g, out_layers, 0, scene->dropout, st, !steady);
        if (rc != TRIPS_OK)
        {
            ctx->have_sizes = false;
            return rc;
        }
        ctx->size_key   = key;
        ctx->have_sizes = true;
    }
    else
    {
        // Nothing is kept for a backward pass: the views are rendered kEvalSubBatch at a time, so the scratch of a call
        // with many views (a batch of 64 evaluation views) is that of kEvalSubBatch views.  The inspection calls then
        // describe the last sub-batch.
        ctx->have_sizes = false;
        for (int b0 = 0; b0 < B; b0 += kEvalSubBatch)
        {
            const int nb = std::min(kEvalSubBatch, B - b0);
            const int rc = forward_views(ctx, scene, views + b0, nb, params, g, out_layers, (size_t)b0,
                                         nullptr, st, true);
            if (rc != TRIPS_OK) return rc;
        }
    }
    ctx->have_forward = true;
    return TRIPS_OK;
}

int trips_backward(TripsContext* ctx, const TripsScene* scene, const float* const* grad_layers, const TripsGrads* grads,
                   void* stream)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    if (!scene || !grad_layers || !grads) return fail(ctx, TRIPS_ERR_INVALID_ARG, "null argument");
    if (!ctx->have_forward || !ctx->params.train) return fail(ctx, TRIPS_ERR_NO_FORWARD, "no training forward pass to differentiate");
    if (scene->n_points != ctx->N || scene->n_tex != ctx->n_tex || scene->channels != ctx->C)
        return fail(ctx, TRIPS_ERR_INVALID_ARG, "scene sizes differ from the forward pass");
    const Geom& g = ctx->geom;
    for (int l = 0; l < g.L; ++l)
        if (!grad_layers[l]) return fail(ctx, TRIPS_ERR_INVALID_ARG, "null gradient layer");
    cudaStream_t st = (cudaStream_t)stream;
    const int B = ctx->B, C = ctx->C;
    const size_t N = (size_t)ctx->N;

    const size_t GS = (size_t)egrad_stride(C);
    CU_CHECK(ctx, ensure(ctx->egrad, sizeof(float) * GS * ctx->entry_cap + 16));  // one row per entry the arrays can hold
    CU_CHECK(ctx, ensure(ctx->g_point, sizeof(float) * GS * N + 16));
    CU_CHECK(ctx, ensure(ctx->g_conf_pt, sizeof(float) * N + 16));
    const size_t small_bytes = sizeof(double) * (TRIPS_MAX_CHANNELS + (size_t)B * 19);  // background | per view: 6 pose, 5 pinhole, 8 distortion
    CU_CHECK(ctx, ensure(ctx->g_small, small_bytes));
    BwdBuffers bb;
    bb.egrad        = (float*)ctx->egrad.p;
    bb.g_point      = (float*)ctx->g_point.p;
    bb.g_conf_pt    = (float*)ctx->g_conf_pt.p;
    bb.g_bg         = (double*)ctx->g_small.p;
    bb.g_pose       = bb.g_bg + TRIPS_MAX_CHANNELS;
    bb.g_k          = bb.g_pose + (size_t)B * 6;
    bb.g_dis        = bb.g_k + (size_t)B * 5;
    ScenePtrs sp  = scene_ptrs(scene);
    FwdBuffers fb = fwd_buffers(ctx);
    // all accumulators start from zero (timed with the gradient bookkeeping of the unpack stage)
    auto clear_accumulators = [&]() -> cudaError_t {
        cudaError_t e = cudaSuccess;
        if (N > 0 && e == cudaSuccess) e = cudaMemsetAsync(ctx->g_point.p, 0, sizeof(float) * GS * N, st);
        if (N > 0 && e == cudaSuccess) e = cudaMemsetAsync(ctx->g_conf_pt.p, 0, sizeof(float) * N, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(ctx->g_small.p, 0, small_bytes, st);
        if (grads->pose_tangent && e == cudaSuccess) e = cudaMemsetAsync(grads->pose_tangent, 0, sizeof(double) * 6 * scene->n_images, st);
        if (grads->intrinsics && e == cudaSuccess) e = cudaMemsetAsync(grads->intrinsics, 0, sizeof(float) * 13 * scene->n_cameras, st);
        if (N > 0 && e == cudaSuccess) e = launch_zero_entry_rows(C, B, fb, bb, ctx->sm_count, st);
        return e;
    };
    STAGE(ctx, TRIPS_STAGE_UNPACK, N > 0 ? 1 : 0, st, clear_accumulators());
    ConstLayerPtrs gin{};
    for (int l = 0; l < g.L; ++l) gin.p[l] = grad_layers[l];
    const bool cam_grads = grads->pose_tangent || grads->intrinsics;
    STAGE(ctx, TRIPS_STAGE_BACKWARD, 1, st,
          launch_blend_backward(sp, (const CamConst*)ctx->cams.p, g, ctx->params, B, fb, bb, gin, cam_grads, ctx->sm_count, st));
    const int n_unpack = (N > 0 ? 2 : 0) + 1;
    STAGE(ctx, TRIPS_STAGE_UNPACK, n_unpack, st,
          launch_unpack_grads(sp, (const CamConst*)ctx->cams.p, B, fb, bb, *grads, ctx->params, ctx->sm_count, st));
    return TRIPS_OK;
}

uint32_t trips_last_status(TripsContext* ctx, void* stream)
{
    if (!ctx || !ctx->stats.p) return 0;
    DevStats s{};
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemcpyAsync(&s, ctx->stats.p, sizeof(s), cudaMemcpyDeviceToHost, st) != cudaSuccess) return 0;
    if (cudaStreamSynchronize(st) != cudaSuccess) return 0;
    unsigned zero = 0;
    cudaMemcpyAsync((char*)ctx->stats.p + offsetof(DevStats, status), &zero, sizeof(unsigned), cudaMemcpyHostToDevice, st);
    cudaStreamSynchronize(st);
    return s.status;
}

int trips_get_stats(TripsContext* ctx, TripsStats* out, void* stream)
{
    (void)stream;
    if (!ctx || !out) return TRIPS_ERR_INVALID_ARG;
    if (!ctx->have_forward) return fail(ctx, TRIPS_ERR_NO_FORWARD, "no forward pass");
    {
        const int rs = resolve_pending(ctx);  // waits for the totals of a call that did not wait for them itself
        if (rs != TRIPS_OK) return rs;
    }
    *out = ctx->host_stats;
    return TRIPS_OK;
}

int trips_adam_step(TripsContext* ctx, const TripsAdamTensor* tensors, int n_tensors, void* stream)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    if (!tensors || n_tensors < 1) return fail(ctx, TRIPS_ERR_INVALID_ARG, "no tensors");
    cudaStream_t st = (cudaStream_t)stream;
    std::vector<int64_t> start(n_tensors + 1, 0);
    for (int i = 0; i < n_tensors; ++i)
    {
        const TripsAdamTensor& t = tensors[i];
        if (t.n < 0 || (t.n > 0 && (!t.weights || !t.gradients || !t.first_moments || !t.second_moments || !t.steps)))
            return fail(ctx, TRIPS_ERR_INVALID_ARG, "null tensor in Adam group");
        start[i + 1] = start[i] + (t.n + kAdamPerBlock - 1) / kAdamPerBlock;
    }
    if (start[n_tensors] >= (1ll << 31)) return fail(ctx, TRIPS_ERR_TOO_LARGE, "too many elements for one Adam launch");
    const size_t tab_bytes   = sizeof(TripsAdamTensor) * n_tensors;
    const size_t tab_aligned = (tab_bytes + 15) & ~(size_t)15;
    CU_CHECK(ctx, ensure(ctx->adam_tab, tab_aligned + sizeof(int64_t) * (n_tensors + 1)));
    CU_CHECK(ctx, cudaMemcpyAsync(ctx->adam_tab.p, tensors, tab_bytes, cudaMemcpyHostToDevice, st));
    CU_CHECK(ctx, cudaMemcpyAsync((char*)ctx->adam_tab.p + tab_aligned, start.data(), sizeof(int64_t) * (n_tensors + 1),
                                  cudaMemcpyHostToDevice, st));
    STAGE(ctx, TRIPS_STAGE_ADAM, 1, st,
          launch_adam((const TripsAdamTensor*)ctx->adam_tab.p, (const int64_t*)((char*)ctx->adam_tab.p + tab_aligned), n_tensors,
                      start[n_tensors], st));
    return TRIPS_OK;
}

int trips_resize_points(TripsContext* ctx, const int64_t* indices_to_remove, int64_t n_remove, int64_t n_points, int64_t n_new,
                        const TripsPointTensor* tensors, int n_tensors, void* stream)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    if (n_points < 0 || n_remove < 0 || n_remove > n_points || n_new < n_points - n_remove) return fail(ctx, TRIPS_ERR_INVALID_ARG, "bad point counts");
    if (n_remove > 0 && !indices_to_remove) return fail(ctx, TRIPS_ERR_INVALID_ARG, "null removal list");
    if (n_tensors < 0 || n_tensors > TRIPS_MAX_POINT_TENSORS || (n_tensors > 0 && !tensors)) return fail(ctx, TRIPS_ERR_INVALID_ARG, "bad tensor table");
    if (n_points >= (1ll << 32) || n_new >= (1ll << 32)) return fail(ctx, TRIPS_ERR_TOO_LARGE, "more than 2^32 points");
    for (int i = 0; i < n_tensors; ++i)
    {
        const TripsPointTensor& t = tensors[i];
        if (t.rows < 1 || (t.elem_bytes != 4 && t.elem_bytes != 8)) return fail(ctx, TRIPS_ERR_INVALID_ARG, "rows >= 1 and 4- or 8-byte elements");
        if ((n_new > 0 && !t.dst) || (n_points > n_remove && !t.src)) return fail(ctx, TRIPS_ERR_INVALID_ARG, "null tensor");
    }
    cudaStream_t st = (cudaStream_t)stream;
    CU_CHECK(ctx, ensure_stats(ctx, st));
    CU_CHECK(ctx, ensure(ctx->resize_scratch, resize_scratch_bytes(n_points)));
    STAGE(ctx, TRIPS_STAGE_RESIZE, 5, st,
          launch_resize_points(indices_to_remove, n_remove, n_points, n_new, tensors, n_tensors, ctx->resize_scratch.p, (DevStats*)ctx->stats.p,
                               ctx->sm_count, st));
    ctx->have_forward = false;  // the scratch of the last forward pass describes the old point set
    return TRIPS_OK;
}

int trips_fused_reduce_adam(TripsContext* ctx, const float* const* grad_ptrs, float* const* param_ptrs, int world, int rank,
                            const TripsAdamSegment* segments, int n_segments, int64_t lo, int64_t hi, float* first_moments,
                            float* second_moments, int32_t* steps, void* stream)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    if (!grad_ptrs || !param_ptrs || !segments) return fail(ctx, TRIPS_ERR_INVALID_ARG, "null argument");
    if (world < 1 || world > TRIPS_MAX_RANKS || rank < 0 || rank >= world) return fail(ctx, TRIPS_ERR_INVALID_ARG, "bad world / rank");
    if (n_segments < 1 || n_segments > TRIPS_MAX_SEGMENTS || segments[0].offset != 0) return fail(ctx, TRIPS_ERR_INVALID_ARG, "bad segment table");
    for (int s = 1; s < n_segments; ++s)
        if (segments[s].offset <= segments[s - 1].offset) return fail(ctx, TRIPS_ERR_INVALID_ARG, "segments must be sorted by offset");
    if (lo < 0 || hi < lo) return fail(ctx, TRIPS_ERR_INVALID_ARG, "bad slice");
    for (int r = 0; r < world; ++r)
        if (!grad_ptrs[r] || !param_ptrs[r] || (((uintptr_t)grad_ptrs[r] | (uintptr_t)param_ptrs[r]) & 15))
            return fail(ctx, TRIPS_ERR_INVALID_ARG, "flat buffers must be non-null and 16-byte aligned");
    if (hi > lo && (!first_moments || !second_moments || !steps)) return fail(ctx, TRIPS_ERR_INVALID_ARG, "null optimizer state");
    cudaStream_t st = (cudaStream_t)stream;
    STAGE(ctx, TRIPS_STAGE_FUSED_ADAM, hi > lo ? 1 : 0, st,
          launch_fused_reduce_adam(grad_ptrs, param_ptrs, world, rank, segments, n_segments, lo, hi, first_moments, second_moments,
                                   steps, ctx->sm_count, st));
    return TRIPS_OK;
}

int trips_fused_reduce_adam_multicast(TripsContext* ctx, const float* grad_multicast, float* param_multicast, const float* param_local,
                                      const TripsAdamSegment* segments, int n_segments, int64_t lo, int64_t hi, float* first_moments,
                                      float* second_moments, int32_t* steps, void* stream)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    if (!grad_multicast || !param_multicast || !param_local || !segments) return fail(ctx, TRIPS_ERR_INVALID_ARG, "null argument");
    if (n_segments < 1 || n_segments > TRIPS_MAX_SEGMENTS || segments[0].offset != 0) return fail(ctx, TRIPS_ERR_INVALID_ARG, "bad segment table");
    for (int s = 1; s < n_segments; ++s)
        if (segments[s].offset <= segments[s - 1].offset) return fail(ctx, TRIPS_ERR_INVALID_ARG, "segments must be sorted by offset");
    if (lo < 0 || hi < lo || ((lo | hi) & 3)) return fail(ctx, TRIPS_ERR_INVALID_ARG, "the slice must start and end on a multiple of 4 elements");
    if (((uintptr_t)grad_multicast | (uintptr_t)param_multicast | (uintptr_t)param_local) & 15)
        return fail(ctx, TRIPS_ERR_INVALID_ARG, "flat buffers must be 16-byte aligned");
    if (hi > lo && (!first_moments || !second_moments || !steps)) return fail(ctx, TRIPS_ERR_INVALID_ARG, "null optimizer state");
    cudaStream_t st = (cudaStream_t)stream;
    STAGE(ctx, TRIPS_STAGE_FUSED_ADAM, hi > lo ? 1 : 0, st,
          launch_fused_multicast_adam(grad_multicast, param_multicast, param_local, segments, n_segments, lo, hi, first_moments,
                                      second_moments, steps, ctx->sm_count, st));
    return TRIPS_OK;
}

int trips_enable_stage_timers(TripsContext* ctx, int enable)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    ctx->timers.enabled = enable != 0;
    return TRIPS_OK;
}

int trips_get_stage_times(TripsContext* ctx, double* ms, int64_t* timed_calls, int64_t* kernel_launches, int reset)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    ctx->timers.collect();
    for (int i = 0; i < TRIPS_NUM_STAGES; ++i)
    {
        if (ms) ms[i] = ctx->timers.ms[i];
        if (timed_calls) timed_calls[i] = ctx->timers.timed[i];
        if (kernel_launches) kernel_launches[i] = ctx->timers.launches[i];
        if (reset)
        {
            ctx->timers.ms[i]       = 0.0;
            ctx->timers.timed[i]    = 0;
            ctx->timers.launches[i] = 0;
        }
    }
    return TRIPS_OK;
}

const char* trips_stage_name(int stage)
{
    static const char* names[TRIPS_NUM_STAGES] = {"setup_cams", "bin_points", "count", "scan", "collect", "sort_blend",
                                                  "blend_backward", "unpack_grads", "adam", "l1_loss", "fused_reduce_adam", "resize_points"};
    return (stage >= 0 && stage < TRIPS_NUM_STAGES) ? names[stage] : "?";
}

int trips_l1_loss_backward(TripsContext* ctx, const float* const* out_layers, const float* const* target_layers,
                           float* const* grad_layers, const int64_t* layer_numel, int num_layers, double* loss_out,
                           void* stream)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    if (!out_layers || !target_layers || !grad_layers || !layer_numel || !loss_out || num_layers < 1 ||
        num_layers > TRIPS_MAX_LAYERS)
        return fail(ctx, TRIPS_ERR_INVALID_ARG, "bad l1 loss arguments");
    cudaStream_t st = (cudaStream_t)stream;
    L1Args a{};
    int64_t total = 0;
    for (int l = 0; l < num_layers; ++l)
    {
        if (!out_layers[l] || !target_layers[l] || !grad_layers[l] || layer_numel[l] < 0)
            return fail(ctx, TRIPS_ERR_INVALID_ARG, "null layer in l1 loss");
        a.out[l]    = out_layers[l];
        a.target[l] = target_layers[l];
        a.grad[l]   = grad_layers[l];
        a.start[l]  = total;
        total += layer_numel[l];
    }
    for (int l = num_layers; l <= TRIPS_MAX_LAYERS; ++l) a.start[l] = total;
    a.L = num_layers;
    CU_CHECK(ctx, cudaMemsetAsync(loss_out, 0, sizeof(double), st));
    STAGE(ctx, TRIPS_STAGE_LOSS, 1, st, launch_l1_loss(a, total, loss_out, ctx->sm_count, st));
    return TRIPS_OK;
}

int trips_debug_points(TripsContext* ctx, int view, float* depth, int32_t* nlayers, float* record, void* stream)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    if (!ctx->have_forward) return fail(ctx, TRIPS_ERR_NO_FORWARD, "no forward pass");
    if (view < 0 || view >= ctx->B) return fail(ctx, TRIPS_ERR_INVALID_ARG, "view out of range");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t N = (size_t)ctx->N, ES = 8;  // the two float4 of an entry's head
    unsigned long long eb[2];
    CU_CHECK(ctx, cudaMemcpyAsync(eb, (unsigned long long*)ctx->entry_base.p + view, sizeof(eb), cudaMemcpyDeviceToHost, st));
    CU_CHECK(ctx, cudaStreamSynchronize(st));
    const size_t n = (size_t)(eb[1] - eb[0]);
    const size_t TS = (size_t)tail_stride(ctx->C);
    std::vector<float> e(n * ES), tl(n * TS);
    if (n)
    {
        CU_CHECK(ctx, cudaMemcpyAsync(e.data(), (float*)ctx->entries.p + eb[0] * ES, sizeof(float) * n * ES, cudaMemcpyDeviceToHost, st));
        CU_CHECK(ctx, cudaMemcpyAsync(tl.data(), (float*)ctx->entries.p + 8 * ctx->entry_cap + eb[0] * TS, sizeof(float) * n * TS,
                                      cudaMemcpyDeviceToHost, st));
    }
    CU_CHECK(ctx, cudaStreamSynchronize(st));
    // the per-point arrays of the reference (depth = -1 for culled points) are rebuilt from the view's entries
    for (size_t i = 0; i < N; ++i)
    {
        if (depth) depth[i] = -1.f;
        if (nlayers) nlayers[i] = 0;
        if (record) record[4 * i] = record[4 * i + 1] = record[4 * i + 2] = record[4 * i + 3] = 0.f;
    }
    for (size_t k = 0; k < n; ++k)
    {
        const float* en = e.data() + k * ES;
        int32_t pid, nl;
        memcpy(&pid, en + 4, 4);
        memcpy(&nl, en + 7, 4);
        nl &= (1 << kRankShift) - 1;  // the spatial rank shares the word
        if (pid < 0 || (size_t)pid >= N) continue;
        if (depth) depth[pid] = en[5];
        if (nlayers) nlayers[pid] = nl;
        if (record)
        {
            record[4 * (size_t)pid + 0] = en[0];
            record[4 * (size_t)pid + 1] = en[1];
            record[4 * (size_t)pid + 2] = en[2];
            record[4 * (size_t)pid + 3] = tl[k * TS + 3];  // texture index
        }
    }
    return TRIPS_OK;
}

int trips_debug_lists(TripsContext* ctx, int view, int32_t* counts, int64_t* offsets, uint64_t* frags, int64_t* n_frags,
                      void* stream)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    if (!ctx->have_forward) return fail(ctx, TRIPS_ERR_NO_FORWARD, "no forward pass");
    if (view < 0 || view >= ctx->B) return fail(ctx, TRIPS_ERR_INVALID_ARG, "view out of range");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t P = (size_t)ctx->geom.P, off = (size_t)view * P;
    unsigned long long vb[2];
    CU_CHECK(ctx, cudaMemcpyAsync(vb, (unsigned long long*)ctx->view_base.p + view, sizeof(vb), cudaMemcpyDeviceToHost, st));
    std::vector<uint32_t> c(P), e(P);
    CU_CHECK(ctx, cudaMemcpyAsync(c.data(), (uint32_t*)ctx->counts.p + off, sizeof(uint32_t) * P, cudaMemcpyDeviceToHost, st));
    CU_CHECK(ctx, cudaMemcpyAsync(e.data(), (uint32_t*)ctx->offsets.p + off, sizeof(uint32_t) * P, cudaMemcpyDeviceToHost, st));
    CU_CHECK(ctx, cudaStreamSynchronize(st));
    const unsigned long long nf = vb[1] - vb[0];
    if (n_frags) *n_frags = (int64_t)nf;
    for (size_t i = 0; i < P; ++i)
    {
        if (counts) counts[i] = (int32_t)c[i];
        if (offsets) offsets[i] = (int64_t)e[i] - (int64_t)c[i];  // the collect pass advanced the offsets to the list ends
    }
    if (frags && nf)
    {
        std::vector<uint4> f(nf);
        CU_CHECK(ctx, cudaMemcpyAsync(f.data(), (uint4*)ctx->frags.p + vb[0], sizeof(uint4) * nf, cudaMemcpyDeviceToHost, st));
        CU_CHECK(ctx, cudaStreamSynchronize(st));
        for (unsigned long long i = 0; i < nf; ++i) frags[i] = ((uint64_t)f[i].y << 32) | f[i].x;
    }
    return TRIPS_OK;
}

int trips_debug_records(TripsContext* ctx, int view, int32_t* nrec, int32_t* rec_pid, float* rec_alpha, void* stream)
{
    if (!ctx) return TRIPS_ERR_INVALID_ARG;
    if (!ctx->have_forward || !ctx->params.train) return fail(ctx, TRIPS_ERR_NO_FORWARD, "no training forward pass");
    if (view < 0 || view >= ctx->B) return fail(ctx, TRIPS_ERR_INVALID_ARG, "view out of range");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t P = (size_t)ctx->geom.P, off = (size_t)view * P;
    std::vector<uint8_t> n(P);
    std::vector<uint2> r(P * 16);
    const size_t ES = 8;  // the two float4 of an entry's head
    unsigned long long eb[2];
    CU_CHECK(ctx, cudaMemcpyAsync(eb, (unsigned long long*)ctx->entry_base.p + view, sizeof(eb), cudaMemcpyDeviceToHost, st));
    CU_CHECK(ctx, cudaMemcpyAsync(n.data(), (uint8_t*)ctx->rec_n.p + off, P, cudaMemcpyDeviceToHost, st));
    CU_CHECK(ctx, cudaMemcpyAsync(r.data(), (uint2*)ctx->records.p + off * 16, sizeof(uint2) * 16 * P, cudaMemcpyDeviceToHost, st));
    CU_CHECK(ctx, cudaStreamSynchronize(st));
    const size_t n_e = (size_t)(eb[1] - eb[0]);
    std::vector<float> e(n_e * ES);
    if (n_e) CU_CHECK(ctx, cudaMemcpyAsync(e.data(), (float*)ctx->entries.p + eb[0] * ES, sizeof(float) * n_e * ES, cudaMemcpyDeviceToHost, st));
    CU_CHECK(ctx, cudaStreamSynchronize(st));
    // records hold the entry index of the fragment's point; report the point id
    for (size_t p = 0; p < P; ++p)
        for (int j = 0; j < n[p]; ++j)
        {
            const uint32_t ei = r[p * 16 + j].x;
            uint32_t pid      = 0xffffffffu;
            if (ei < n_e) memcpy(&pid, e.data() + (size_t)ei * ES + 4, 4);
            r[p * 16 + j].x = pid;
        }
    for (size_t p = 0; p < P; ++p)
    {
        if (nrec) nrec[p] = n[p];
        for (int j = 0; j < 16; ++j)
        {
            const bool present = j < n[p];
            if (rec_pid) rec_pid[p * 16 + j] = present ? (int32_t)r[p * 16 + j].x : -1;
            if (rec_alpha)
            {
                float a;
                memcpy(&a, &r[p * 16 + j].y, 4);
                rec_alpha[p * 16 + j] = present ? a : -1.f;
            }
        }
    }
    return TRIPS_OK;
}

}  // extern "C"
