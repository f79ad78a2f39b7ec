// C ABI of the library: parameter validation, workspace layout and launch sequencing.
// No kernel lives here; see voxelize.cu, rulebook.cu, conv_simt.cu, conv_umma.cu, sparse2dense.cu.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"

namespace sessd {

std::atomic<uint64_t> g_launches{0};
thread_local StageRecorder* g_recorder = nullptr;
static thread_local std::string t_last_error;

void set_cuda_error(cudaError_t e, const char* what) {
    t_last_error = std::string(cudaGetErrorName(e)) + ": " + cudaGetErrorString(e) + " in " + what;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

void StageRecorder::before(cudaStream_t s) {
    cudaEvent_t e;
    cudaEventCreate(&e);
    cudaEventRecord(e, s);
    events.push_back(e);
}
void StageRecorder::after(const char* name, cudaStream_t s) {
    cudaEvent_t e;
    cudaEventCreate(&e);
    cudaEventRecord(e, s);
    events.push_back(e);
    names.push_back(name);
}

int launch_rulebook_export(const int32_t* nbr, const int32_t* out_num, int frame, int kvol, int max_voxels,
                           int32_t* pairs, uint32_t* pair_num, cudaStream_t stream);
int launch_count_pairs(const int32_t* nbr, const int32_t* out_num, int batch, int max_voxels, int kvol,
                       unsigned long long* total, cudaStream_t stream);

namespace {

constexpr int kStatusInts = 256;  // status block: 1 KB; word 0 is the status, bytes 256.. hold 64 pair counters

// np.round as the reference mimics it (voxelGenerator.cu:61-68).
int np_round_f32(float x) {
    const int x2 = (int)(x * 2.0f);
    if (x != (float)(int)x && (float)x2 == x * 2.0f) return (int)(x / 2.0f + 0.5f) * 2;
    return (int)(x + 0.5f);
}

bool voxel_params_ok(const sessd_voxel_params* p, int batch, int max_points) {
    if (p->max_voxels < 1 || p->max_points_per_voxel < 1 || p->max_points_per_voxel > 8) return false;
    if (p->voxel_feature_num != 4 || p->point_feature_num != 4) return false;
    if (!(p->voxel_x > 0.f) || !(p->voxel_y > 0.f) || !(p->voxel_z > 0.f)) return false;
    if (p->grid_x < 1 || p->grid_y < 1 || p->grid_z < 1) return false;
    if ((uint64_t)p->grid_x * p->grid_y * p->grid_z >= 0xFFFFFFFFull) return false;
    if (batch < 1 || batch > kMaxBatch || max_points < 1 || max_points > (1 << 28)) return false;
    if ((uint64_t)batch * p->max_voxels > 0x7FFFFFFFull) return false;
    return true;
}

bool is_subm_333(const ConvGeom& g) {
    return g.kvol == 27 && g.K[0] == 3 && g.K[1] == 3 && g.K[2] == 3 && g.P[0] == 1 && g.P[1] == 1 && g.P[2] == 1;
}

struct ConvWorkspace {
    int32_t* status;
    void* ones_base;      // tables: every word 0xFFFFFFFF before use
    size_t ones_bytes;
    Buckets buckets;      // submanifold 3x3x3: x-grouped table of the input coordinates
    Table in_table;       // other submanifold geometries: flat table of the input coordinates
    BitGrid out_bits;     // strided: occupancy grid of the output level
    void* zero_base;      // occupancy grid + tile masks: zero before use
    size_t zero_bytes;
    uint32_t* tile_mask;  // [B][tiles]
    int32_t* chunk_counts;
    int32_t* nbr;
};

void conv_workspace_layout(Bump& bump, const sessd_conv_params* p, const ConvGeom& g, int batch, ConvWorkspace* w) {
    *w = ConvWorkspace{};
    w->status = bump.take<int32_t>(kStatusInts);
    const uint32_t cap = pow2_at_least(2ull * (uint64_t)p->max_voxels);
    const size_t per = (size_t)batch * cap;
    const int shift = 32 - ilog2(cap);
    if (p->subm && is_subm_333(g)) {
        const uint32_t capb = pow2_at_least((uint64_t)p->max_voxels);
        w->buckets = Buckets{bump.take<uint32_t>((size_t)batch * capb * 8), capb, 32 - ilog2(capb)};
        w->ones_base = w->buckets.data;
        w->ones_bytes = (size_t)batch * capb * 8 * sizeof(uint32_t);
    } else if (p->subm) {
        uint32_t* block = bump.take<uint32_t>(per * 2);
        w->in_table = Table{block, nullptr, reinterpret_cast<int32_t*>(block ? block + per : nullptr), cap, shift, 1, 1};
        w->ones_base = block;
        w->ones_bytes = per * 2 * sizeof(uint32_t);
    } else {
        w->out_bits = bitgrid_shape(g.out_shape);
        w->chunk_counts = bump.take<int32_t>((size_t)batch * w->out_bits.chunks);
    }
    // occupancy grid (strided layers) and tile masks in one block, reset to zero by a single fill
    const size_t tiles = (size_t)(p->max_voxels + 127) / 128;
    const size_t mask_bytes = (batch * tiles * sizeof(uint32_t) + 15) / 16 * 16;
    const size_t grid_bytes = p->subm ? 0 : (size_t)batch * w->out_bits.words * sizeof(uint4);
    char* zero = bump.take<char>(grid_bytes + mask_bytes);
    w->zero_base = zero;
    w->zero_bytes = grid_bytes + mask_bytes;
    w->out_bits.rec = reinterpret_cast<uint4*>(zero);
    w->tile_mask = reinterpret_cast<uint32_t*>(zero ? zero + grid_bytes : nullptr);
    w->nbr = bump.take<int32_t>((size_t)batch * nbr_frame_words(g.kvol, p->max_voxels));
}

bool conv_params_ok(const sessd_conv_params* p, int batch) {
    if (p->in_channel < 1 || p->out_channel < 1 || p->max_voxels < 1) return false;
    if (batch < 1 || batch > kMaxBatch) return false;
    if ((uint64_t)batch * p->max_voxels * 27ull > 0x7FFFFFFFull) return false;
    return true;
}

size_t esize(int dtype) { return dtype == SESSD_F32 ? 4 : 2; }

int choose_conv(const ConvLaunch& c_in, cudaStream_t stream) {
    const ConvLaunch& c = c_in;
    if (c.dtype == SESSD_F16 && conv_umma_supported(c.cin, c.cout) && c.umma_weights) return launch_conv_umma(c, stream);
    return launch_conv_simt(c, stream);
}

}  // namespace
}  // namespace sessd

using namespace sessd;

struct sessd_conv_weights {
    sessd_conv_weights_impl impl;
};

struct sessd_backbone {
    sessd_voxel_params vp;
    sessd_s2d_params s2d;
    bool has_s2d;
    sessd_pad2d_params pad;   // zero border folded into the dense output (all zero by default)
    int dtype;
    struct Layer {
        sessd_conv_params p;
        ConvGeom g;
        sessd_conv_weights* w;
        int level_in, level_out;
    };
    std::vector<Layer> layers;
    int nlevels;
    std::vector<int> level_shape;  // 3 ints per level
    std::vector<char> level_has_subm;
    int max_voxels;
    int kvol_strided_max, ncand_max;
};

namespace {

struct BackboneWorkspace {
    int32_t* status;
    VoxelWorkspace vox;
    void* voxel_feat;
    std::vector<int32_t*> coors, num;
    std::vector<BitGrid> bits;       // occupancy grids of the derived levels (index 0 unused)
    Buckets buckets0;                // x-grouped table of the voxeliser's rows (level 0)
    void* ones_base;
    size_t ones_bytes;
    std::vector<int32_t*> nbr_subm;
    std::vector<uint32_t*> mask_subm;     // per level
    std::vector<uint32_t*> mask_layer;    // per strided layer (indexed by layer)
    void* zero_base;
    size_t zero_bytes;
    int32_t* nbr_strided;
    int32_t* chunk_counts;
    std::vector<void*> feat;
};

void backbone_layout(Bump& bump, const sessd_backbone* bb, int batch, int max_points, BackboneWorkspace* w) {
    const int maxV = bb->max_voxels;
    w->status = bump.take<int32_t>(kStatusInts);
    voxel_workspace_layout(bump, &bb->vp, batch, max_points, &w->vox);
    w->vox.status = w->status;
    w->voxel_feat = bump.take<char>((size_t)batch * maxV * 4 * esize(bb->dtype));
    w->coors.assign(bb->nlevels, nullptr);
    w->num.assign(bb->nlevels, nullptr);
    w->bits.assign(bb->nlevels, BitGrid{});
    w->nbr_subm.assign(bb->nlevels, nullptr);
    w->mask_subm.assign(bb->nlevels, nullptr);
    w->mask_layer.assign(bb->layers.size(), nullptr);
    for (int l = 0; l < bb->nlevels; ++l) {
        w->coors[l] = bump.take<int32_t>((size_t)batch * maxV * 4);
        w->num[l] = bump.take<int32_t>(batch);
    }
    // the x-grouped table of level 0, reset to 0xFF by one fill (the voxeliser resets its own table)
    const uint32_t capb = pow2_at_least((uint64_t)maxV);
    const size_t perb = (size_t)batch * capb * 8;
    uint32_t* block = bump.take<uint32_t>(perb + 4);
    w->buckets0 = Buckets{block, capb, 32 - ilog2(capb)};
    w->ones_base = block;
    w->ones_bytes = perb * sizeof(uint32_t);
    // occupancy grids of the derived levels and all tile masks in one block, reset to zero by one fill
    const size_t tiles = (size_t)(maxV + 127) / 128;
    const size_t mask_words = (batch * tiles + 3) / 4 * 4;
    size_t nmasks = 0;
    for (int l = 0; l < bb->nlevels; ++l) nmasks += bb->level_has_subm[l] ? 1 : 0;
    for (auto& L : bb->layers) nmasks += L.p.subm ? 0 : 1;
    size_t grid_recs = 0;
    int chunks_max = 1;
    for (int l = 1; l < bb->nlevels; ++l) {
        w->bits[l] = bitgrid_shape(&bb->level_shape[3 * l]);
        grid_recs += (size_t)batch * w->bits[l].words;
        if (w->bits[l].chunks > chunks_max) chunks_max = w->bits[l].chunks;
    }
    char* zero = bump.take<char>(grid_recs * sizeof(uint4) + mask_words * nmasks * sizeof(uint32_t) + 16);
    w->zero_base = zero;
    w->zero_bytes = grid_recs * sizeof(uint4) + mask_words * nmasks * sizeof(uint32_t);
    size_t off = 0;
    for (int l = 1; l < bb->nlevels; ++l) {
        w->bits[l].rec = reinterpret_cast<uint4*>(zero ? zero + off : nullptr);
        off += (size_t)batch * w->bits[l].words * sizeof(uint4);
    }
    uint32_t* masks = reinterpret_cast<uint32_t*>(zero ? zero + off : nullptr);
    size_t mi = 0;
    for (int l = 0; l < bb->nlevels; ++l)
        if (bb->level_has_subm[l]) w->mask_subm[l] = masks ? masks + mask_words * mi++ : (mi++, nullptr);
    for (size_t i = 0; i < bb->layers.size(); ++i)
        if (!bb->layers[i].p.subm) w->mask_layer[i] = masks ? masks + mask_words * mi++ : (mi++, nullptr);
    for (int l = 0; l < bb->nlevels; ++l)
        if (bb->level_has_subm[l]) w->nbr_subm[l] = bump.take<int32_t>((size_t)batch * nbr_frame_words(27, maxV));
    w->nbr_strided =
        bump.take<int32_t>((size_t)batch * nbr_frame_words(bb->kvol_strided_max > 0 ? bb->kvol_strided_max : 1, maxV));
    w->chunk_counts = bump.take<int32_t>((size_t)batch * chunks_max);
    w->feat.assign(bb->layers.size(), nullptr);
    for (size_t i = 0; i < bb->layers.size(); ++i)
        w->feat[i] = bump.take<char>((size_t)batch * maxV * bb->layers[i].p.out_channel * esize(bb->dtype));
}

}  // namespace

extern "C" {

const char* sessd_version(void) { return "sessd-b200 0.1 (sm_100a)"; }

int sessd_conv_weights_debug_withhold(sessd_conv_weights* w, int on) {
    if (!w) return SESSD_ERR_NULL;
    w->impl.debug_withhold = on ? 1 : 0;
    return SESSD_OK;
}
const char* sessd_last_cuda_error(void) { return t_last_error.c_str(); }
uint64_t sessd_launch_count(void) { return g_launches.load(); }

int sessd_read_status(const void* workspace, void* stream) {
    if (!workspace) return SESSD_ERR_NULL;
    int32_t v = 0;
    SESSD_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    SESSD_CUDA(cudaMemcpy(&v, workspace, sizeof(v), cudaMemcpyDeviceToHost));
    return v & 0x7FFFFFFF;
}

// ---- profiling hooks ------------------------------------------------------------------------

int sessd_profile_begin(void) {
    if (g_recorder) return SESSD_ERR_PARAM;
    g_recorder = new StageRecorder();
    return SESSD_OK;
}

int sessd_profile_end(void* stream, char* names, size_t names_cap, float* ms, int cap) {
    if (!g_recorder) return SESSD_ERR_PARAM;
    StageRecorder* r = g_recorder;
    g_recorder = nullptr;
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    cudaDeviceSynchronize();
    const int n = (int)r->names.size();
    std::string joined;
    for (int i = 0; i < n; ++i) {
        float t = 0.f;
        cudaEventElapsedTime(&t, r->events[2 * i], r->events[2 * i + 1]);
        if (ms && i < cap) ms[i] = t;
        joined += r->names[i];
        joined += '\n';
    }
    for (cudaEvent_t e : r->events) cudaEventDestroy(e);
    if (names && names_cap > 0) {
        std::strncpy(names, joined.c_str(), names_cap - 1);
        names[names_cap - 1] = 0;
    }
    delete r;
    return n;
}

// ---- voxel generator ------------------------------------------------------------------------

int sessd_voxel_configure(sessd_voxel_params* p) {
    if (!p) return SESSD_ERR_NULL;
    if (!(p->voxel_x > 0.f) || !(p->voxel_y > 0.f) || !(p->voxel_z > 0.f)) return SESSD_ERR_PARAM;
    p->grid_x = np_round_f32((p->x_max - p->x_min) / p->voxel_x);
    p->grid_y = np_round_f32((p->y_max - p->y_min) / p->voxel_y);
    p->grid_z = np_round_f32((p->z_max - p->z_min) / p->voxel_z);
    return SESSD_OK;
}

size_t sessd_voxelize_workspace_bytes(const sessd_voxel_params* p, int batch, int max_points) {
    if (!p || !voxel_params_ok(p, batch, max_points)) return 0;
    Bump bump(nullptr);
    bump.take<int32_t>(kStatusInts);
    VoxelWorkspace w;
    voxel_workspace_layout(bump, p, batch, max_points, &w);
    return bump.total();
}

void* sessd_voxelize_num_points(const sessd_voxel_params* p, int batch, int max_points, void* workspace) {
    if (!p || !workspace || !voxel_params_ok(p, batch, max_points)) return nullptr;
    Bump bump(workspace);
    bump.take<int32_t>(kStatusInts);
    VoxelWorkspace w;
    voxel_workspace_layout(bump, p, batch, max_points, &w);
    return w.num_points;
}

int sessd_voxelize_enqueue(const sessd_voxel_params* p, int batch, int max_points, int out_dtype,
                           const void* const* inputs, void* const* outputs, void* workspace, size_t workspace_bytes,
                           void* stream_) {
    if (!p || !inputs || !outputs || !workspace) return SESSD_ERR_NULL;
    if (!inputs[0] || !inputs[1] || !outputs[0] || !outputs[1] || !outputs[2]) return SESSD_ERR_NULL;
    if (!voxel_params_ok(p, batch, max_points)) return SESSD_ERR_PARAM;
    if (out_dtype != SESSD_F32 && out_dtype != SESSD_F16) return SESSD_ERR_PARAM;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    Bump bump(workspace);
    int32_t* status = bump.take<int32_t>(kStatusInts);
    VoxelWorkspace w;
    voxel_workspace_layout(bump, p, batch, max_points, &w);
    if (bump.total() > workspace_bytes) return SESSD_ERR_WORKSPACE;
    if (!workspace_aligned(workspace)) return SESSD_ERR_PARAM;
    w.status = status;
    SESSD_CUDA(cudaMemsetAsync(status, 0, kStatusInts * sizeof(int32_t), stream));
    return voxelize_run(p, batch, max_points, out_dtype, static_cast<const float*>(inputs[0]),
                        static_cast<const int32_t*>(inputs[1]), outputs[0], static_cast<int32_t*>(outputs[1]),
                        static_cast<int32_t*>(outputs[2]), w, /*zero_tail=*/true, stream);
}

// ---- sparse convolutions --------------------------------------------------------------------

int sessd_conv_weights_create(const sessd_conv_params* p, const float* weights, const float* scale, const float* shift,
                              int relu, int dtype, sessd_conv_weights** out) {
    if (!p || !weights || !out) return SESSD_ERR_NULL;
    if (dtype != SESSD_F32 && dtype != SESSD_F16) return SESSD_ERR_PARAM;
    ConvGeom g;
    int rc = conv_geom_from_params(p, &g);
    if (rc) return rc;
    if (!conv_simt_supported(p->in_channel, p->out_channel)) return SESSD_ERR_UNSUPPORTED;
    auto* w = new sessd_conv_weights();
    std::memset(&w->impl, 0, sizeof(w->impl));
    w->impl.relu = relu ? 1 : 0;
    w->impl.dtype = dtype;
    w->impl.kvol = g.kvol;
    w->impl.cin = p->in_channel;
    w->impl.cout = p->out_channel;
    const size_t count = (size_t)g.kvol * p->in_channel * p->out_channel;
    auto fail = [&](cudaError_t e, const char* what) {
        set_cuda_error(e, what);
        sessd_conv_weights_destroy(w);
        return SESSD_ERR_CUDA;
    };
    cudaError_t e = cudaMalloc(&w->impl.w, count * esize(dtype));
    if (e != cudaSuccess) return fail(e, "cudaMalloc(weights)");
    if (dtype == SESSD_F32) {
        e = cudaMemcpy(w->impl.w, weights, count * 4, cudaMemcpyHostToDevice);
    } else {
        std::vector<__half> h(count);
        for (size_t i = 0; i < count; ++i) h[i] = __float2half_rn(weights[i]);
        e = cudaMemcpy(w->impl.w, h.data(), count * 2, cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) return fail(e, "cudaMemcpy(weights)");
    if (scale) {
        e = cudaMalloc(&w->impl.scale, p->out_channel * 4);
        if (e != cudaSuccess) return fail(e, "cudaMalloc(scale)");
        e = cudaMemcpy(w->impl.scale, scale, p->out_channel * 4, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) return fail(e, "cudaMemcpy(scale)");
        e = cudaMalloc(&w->impl.shift, p->out_channel * 4);
        if (e != cudaSuccess) return fail(e, "cudaMalloc(shift)");
        if (shift)
            e = cudaMemcpy(w->impl.shift, shift, p->out_channel * 4, cudaMemcpyHostToDevice);
        else
            e = cudaMemset(w->impl.shift, 0, p->out_channel * 4);
        if (e != cudaSuccess) return fail(e, "cudaMemcpy(shift)");
    }
    for (int c = 0; c < 64; ++c) {
        w->impl.host_scale[c] = (scale && c < p->out_channel) ? scale[c] : 1.f;
        w->impl.host_shift[c] = (scale && shift && c < p->out_channel) ? shift[c] : 0.f;
    }
    if (dtype == SESSD_F16 && conv_umma_supported(p->in_channel, p->out_channel)) {
        rc = conv_umma_pack_weights(weights, g.kvol, p->in_channel, p->out_channel, &w->impl.umma_w);
        if (rc) {
            sessd_conv_weights_destroy(w);
            return rc;
        }
    }
    *out = w;
    return SESSD_OK;
}

void sessd_conv_weights_destroy(sessd_conv_weights* w) {
    if (!w) return;
    if (w->impl.w) cudaFree(w->impl.w);
    if (w->impl.scale) cudaFree(w->impl.scale);
    if (w->impl.shift) cudaFree(w->impl.shift);
    if (w->impl.umma_w) cudaFree(w->impl.umma_w);
    delete w;
}

size_t sessd_conv_workspace_bytes(const sessd_conv_params* p, int batch) {
    if (!p || !conv_params_ok(p, batch)) return 0;
    ConvGeom g;
    if (conv_geom_from_params(p, &g)) return 0;
    Bump bump(nullptr);
    ConvWorkspace w;
    conv_workspace_layout(bump, p, g, batch, &w);
    return bump.total();
}

static int conv_enqueue_common(const sessd_conv_params* p, const sessd_conv_weights* w, int batch,
                               const void* const* inputs, void* const* outputs, void* workspace,
                               size_t workspace_bytes, void* stream_, bool subm) {
    if (!p || !w || !inputs || !outputs || !workspace) return SESSD_ERR_NULL;
    if (!inputs[0] || !inputs[1] || !inputs[2] || !outputs[0]) return SESSD_ERR_NULL;
    if (!subm && (!outputs[1] || !outputs[2])) return SESSD_ERR_NULL;
    if (!conv_params_ok(p, batch) || (p->subm != 0) != subm) return SESSD_ERR_PARAM;
    ConvGeom g;
    int rc = conv_geom_from_params(p, &g);
    if (rc) return rc;
    if (w->impl.cin != p->in_channel || w->impl.cout != p->out_channel || w->impl.kvol != g.kvol) return SESSD_ERR_PARAM;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    Bump bump(workspace);
    ConvWorkspace ws;
    conv_workspace_layout(bump, p, g, batch, &ws);
    if (bump.total() > workspace_bytes) return SESSD_ERR_WORKSPACE;
    if (!workspace_aligned(workspace)) return SESSD_ERR_PARAM;
    const int maxV = p->max_voxels;
    const int32_t* in_coors = static_cast<const int32_t*>(inputs[1]);
    const int32_t* in_num = static_cast<const int32_t*>(inputs[2]);
    SESSD_CUDA(cudaMemsetAsync(ws.status, 0, kStatusInts * sizeof(int32_t), stream));
    if (ws.ones_bytes) {
        rc = launch_fill_ones(ws.ones_base, ws.ones_bytes, stream);
        if (rc) return rc;
    }
    rc = launch_fill_zero(ws.zero_base, ws.zero_bytes, stream);
    if (rc) return rc;
    const int32_t* out_num = in_num;
    if (subm && is_subm_333(g)) {
        rc = launch_bucket_build(in_coors, in_num, batch, maxV, g.in_shape, ws.buckets, ws.status, stream);
        if (rc) return rc;
        rc = launch_nbr_build_subm(in_coors, in_num, batch, maxV, g.in_shape, ws.buckets, ws.nbr, ws.tile_mask, stream);
        if (rc) return rc;
    } else if (subm) {
        rc = launch_table_build(in_coors, in_num, batch, maxV, g.in_shape, ws.in_table, ws.status, stream);
        if (rc) return rc;
        rc = launch_nbr_build(in_coors, in_num, batch, maxV, g, ws.in_table, ws.nbr, stream);
        if (rc) return rc;
        rc = launch_tile_mask(ws.nbr, in_num, batch, maxV, g.kvol, ws.tile_mask, stream);
        if (rc) return rc;
    } else {
        rc = launch_mark_outputs(in_coors, in_num, batch, maxV, g, ws.out_bits, stream);
        if (rc) return rc;
        rc = launch_number_outputs(ws.out_bits, batch, maxV, ws.chunk_counts, static_cast<int32_t*>(outputs[1]),
                                   static_cast<int32_t*>(outputs[2]), ws.status, stream);
        if (rc) return rc;
        out_num = static_cast<const int32_t*>(outputs[2]);
        // the caller's input rows come in any order and have no grid of their own: input-stationary map
        rc = launch_scatter_rows(in_coors, in_num, out_num, batch, maxV, g, ws.out_bits, ws.nbr, ws.tile_mask, stream);
        if (rc) return rc;
    }
    ConvLaunch c{};
    c.in = inputs[0];
    c.out = outputs[0];
    c.nbr = ws.nbr;
    c.tile_mask = ws.tile_mask;
    c.out_num = out_num;
    c.weights = w->impl.w;
    c.umma_weights = w->impl.umma_w;
    c.scale = w->impl.scale;
    c.shift = w->impl.shift;
    c.relu = w->impl.relu;
    c.batch = batch;
    c.max_voxels = maxV;
    c.kvol = g.kvol;
    c.cin = p->in_channel;
    c.cout = p->out_channel;
    c.dtype = w->impl.dtype;
    c.status = ws.status;
    c.debug_withhold_weights = w->impl.debug_withhold;
    c.scale_host = w->impl.host_scale;
    c.shift_host = w->impl.host_shift;
    rc = choose_conv(c, stream);
    if (rc) return rc;
    // Rows past the active count are zero in the reference (outputs are memset, submConv3dlayer.cu:594).
    rc = launch_zero_tail(outputs[0], (int)(p->out_channel * esize(w->impl.dtype)), out_num, batch, maxV, stream);
    if (rc) return rc;
    if (!subm) rc = launch_zero_tail(outputs[1], 16, out_num, batch, maxV, stream);
    return rc;
}

int sessd_subm_conv_enqueue(const sessd_conv_params* p, const sessd_conv_weights* w, int batch,
                            const void* const* inputs, void* const* outputs, void* workspace, size_t workspace_bytes,
                            void* stream) {
    return conv_enqueue_common(p, w, batch, inputs, outputs, workspace, workspace_bytes, stream, true);
}

int sessd_sparse_conv_enqueue(const sessd_conv_params* p, const sessd_conv_weights* w, int batch,
                              const void* const* inputs, void* const* outputs, void* workspace, size_t workspace_bytes,
                              void* stream) {
    return conv_enqueue_common(p, w, batch, inputs, outputs, workspace, workspace_bytes, stream, false);
}

int sessd_conv_rulebook_export(const sessd_conv_params* p, int batch, int frame, void* workspace,
                               int32_t* indice_pairs, uint32_t* indice_num, void* stream, const void* out_voxel_num) {
    if (!p || !workspace || !indice_pairs || !indice_num || !out_voxel_num) return SESSD_ERR_NULL;
    if (!conv_params_ok(p, batch) || frame < 0 || frame >= batch) return SESSD_ERR_PARAM;
    ConvGeom g;
    int rc = conv_geom_from_params(p, &g);
    if (rc) return rc;
    Bump bump(workspace);
    ConvWorkspace ws;
    conv_workspace_layout(bump, p, g, batch, &ws);
    return launch_rulebook_export(ws.nbr, static_cast<const int32_t*>(out_voxel_num), frame, g.kvol, p->max_voxels,
                                  indice_pairs, indice_num, static_cast<cudaStream_t>(stream));
}

// ---- sparse -> dense -------------------------------------------------------------------------

int sessd_sparse2dense_enqueue(const sessd_s2d_params* p, int batch, int max_voxels, int dtype,
                               const void* const* inputs, void* const* outputs, void* workspace,
                               size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    if (!p || !inputs || !outputs) return SESSD_ERR_NULL;
    if (!inputs[0] || !inputs[1] || !inputs[2] || !outputs[0]) return SESSD_ERR_NULL;
    if (batch < 1 || batch > kMaxBatch || max_voxels < 1 || p->feature_map_channel < 1 || p->feature_map_size_x < 1 ||
        p->feature_map_size_y < 1 || p->feature_map_size_z < 1)
        return SESSD_ERR_PARAM;
    if (dtype != SESSD_F32 && dtype != SESSD_F16) return SESSD_ERR_PARAM;
    return launch_sparse2dense(inputs[0], static_cast<const int32_t*>(inputs[1]), static_cast<const int32_t*>(inputs[2]),
                               batch, max_voxels, p->feature_map_channel, p->feature_map_size_z, p->feature_map_size_y,
                               p->feature_map_size_x, 0, 0, 0, 0, dtype, outputs[0], static_cast<cudaStream_t>(stream));
}

static bool pad_ok(const sessd_pad2d_params* p) {
    return p->top >= 0 && p->bottom >= 0 && p->left >= 0 && p->right >= 0 && p->top < 4096 && p->bottom < 4096 &&
           p->left < 4096 && p->right < 4096;
}

int sessd_sparse2dense_padded_enqueue(const sessd_s2d_params* p, const sessd_pad2d_params* pad, int batch,
                                      int max_voxels, int dtype, const void* const* inputs, void* const* outputs,
                                      void* stream) {
    if (!p || !pad || !inputs || !outputs) return SESSD_ERR_NULL;
    if (!inputs[0] || !inputs[1] || !inputs[2] || !outputs[0]) return SESSD_ERR_NULL;
    if (batch < 1 || batch > kMaxBatch || max_voxels < 1 || p->feature_map_channel < 1 || p->feature_map_size_x < 1 ||
        p->feature_map_size_y < 1 || p->feature_map_size_z < 1 || !pad_ok(pad))
        return SESSD_ERR_PARAM;
    if (dtype != SESSD_F32 && dtype != SESSD_F16) return SESSD_ERR_PARAM;
    return launch_sparse2dense(inputs[0], static_cast<const int32_t*>(inputs[1]), static_cast<const int32_t*>(inputs[2]),
                               batch, max_voxels, p->feature_map_channel, p->feature_map_size_z, p->feature_map_size_y,
                               p->feature_map_size_x, pad->top, pad->bottom, pad->left, pad->right, dtype, outputs[0],
                               static_cast<cudaStream_t>(stream));
}

int sessd_zero_pad2d_enqueue(const sessd_pad2d_params* pad, int batch, int channels, int height, int width, int dtype,
                             const void* const* inputs, void* const* outputs, void* stream) {
    if (!pad || !inputs || !outputs || !inputs[0] || !outputs[0]) return SESSD_ERR_NULL;
    if (batch < 1 || batch > kMaxBatch || channels < 1 || height < 1 || width < 1 || !pad_ok(pad)) return SESSD_ERR_PARAM;
    if (dtype != SESSD_F32 && dtype != SESSD_F16) return SESSD_ERR_PARAM;
    return launch_zero_pad2d(inputs[0], outputs[0], (size_t)batch * channels, height, width, pad->top, pad->bottom,
                             pad->left, pad->right, dtype, static_cast<cudaStream_t>(stream));
}

// ---- whole front end -------------------------------------------------------------------------

int sessd_backbone_create(const sessd_voxel_params* vp, const sessd_conv_params* layers, int nlayers,
                          const float* const* weights, const float* const* scale, const float* const* shift,
                          const sessd_s2d_params* s2d, int dtype, sessd_backbone** out) {
    if (!vp || !layers || !weights || !out) return SESSD_ERR_NULL;
    if (nlayers < 1 || nlayers > 64) return SESSD_ERR_PARAM;
    if (dtype != SESSD_F32 && dtype != SESSD_F16) return SESSD_ERR_PARAM;
    if (!voxel_params_ok(vp, 1, 1)) return SESSD_ERR_PARAM;
    auto* bb = new sessd_backbone();
    bb->vp = *vp;
    bb->has_s2d = s2d != nullptr;
    if (s2d) bb->s2d = *s2d;
    bb->pad = sessd_pad2d_params{0, 0, 0, 0};
    bb->dtype = dtype;
    bb->max_voxels = vp->max_voxels;
    bb->nlevels = 1;
    bb->kvol_strided_max = 0;
    bb->ncand_max = 0;
    bb->level_has_subm.assign(1, 0);
    int rc = SESSD_OK;
    int cur_c = vp->voxel_feature_num;
    for (int i = 0; i < nlayers && rc == SESSD_OK; ++i) {
        sessd_backbone::Layer L{};
        L.p = layers[i];
        L.w = nullptr;
        rc = conv_geom_from_params(&L.p, &L.g);
        if (rc) break;
        if (L.p.max_voxels != bb->max_voxels || L.p.in_channel != cur_c || !weights[i]) { rc = SESSD_ERR_PARAM; break; }
        if (i == 0) {
            // Level 0 keys come from the voxeliser: (z*gy + y)*gx + x must be the layer's own key.
            if (L.g.in_shape[1] != vp->grid_y || L.g.in_shape[2] != vp->grid_x || L.g.in_shape[0] < vp->grid_z) {
                rc = SESSD_ERR_PARAM;
                break;
            }
            bb->level_shape = {L.g.in_shape[0], L.g.in_shape[1], L.g.in_shape[2]};
        }
        const int* shp = &bb->level_shape[3 * (bb->nlevels - 1)];
        if (L.g.in_shape[0] != shp[0] || L.g.in_shape[1] != shp[1] || L.g.in_shape[2] != shp[2]) { rc = SESSD_ERR_PARAM; break; }
        L.level_in = bb->nlevels - 1;
        if (L.p.subm) {
            if (L.g.kvol != 27 || L.g.P[0] != 1 || L.g.P[1] != 1 || L.g.P[2] != 1) { rc = SESSD_ERR_UNSUPPORTED; break; }
            L.level_out = L.level_in;
            bb->level_has_subm[L.level_in] = 1;
        } else {
            L.level_out = bb->nlevels++;
            bb->level_shape.insert(bb->level_shape.end(), {L.g.out_shape[0], L.g.out_shape[1], L.g.out_shape[2]});
            bb->level_has_subm.push_back(0);
            if (L.g.kvol > bb->kvol_strided_max) bb->kvol_strided_max = L.g.kvol;
            if (L.g.ncand > bb->ncand_max) bb->ncand_max = L.g.ncand;
        }
        rc = sessd_conv_weights_create(&L.p, weights[i], scale ? scale[i] : nullptr, shift ? shift[i] : nullptr, 1, dtype,
                                       &L.w);
        if (rc) break;
        cur_c = L.p.out_channel;
        bb->layers.push_back(L);
    }
    if (rc == SESSD_OK && s2d) {
        const sessd_backbone::Layer& last = bb->layers.back();
        if (s2d->feature_map_channel != last.p.out_channel || s2d->feature_map_size_z != last.g.out_shape[0] ||
            s2d->feature_map_size_y != last.g.out_shape[1] || s2d->feature_map_size_x != last.g.out_shape[2])
            rc = SESSD_ERR_PARAM;
    }
    if (rc) {
        sessd_backbone_destroy(bb);
        return rc;
    }
    *out = bb;
    return SESSD_OK;
}

void sessd_backbone_destroy(sessd_backbone* bb) {
    if (!bb) return;
    for (auto& L : bb->layers) sessd_conv_weights_destroy(L.w);
    delete bb;
}

size_t sessd_backbone_workspace_bytes(const sessd_backbone* bb, int batch, int max_points) {
    if (!bb || !voxel_params_ok(&bb->vp, batch, max_points)) return 0;
    if ((uint64_t)batch * bb->max_voxels * 27ull > 0x7FFFFFFFull) return 0;
    Bump bump(nullptr);
    BackboneWorkspace w;
    backbone_layout(bump, bb, batch, max_points, &w);
    return bump.total();
}

static int backbone_enqueue_impl(const sessd_backbone* bb, int batch, int max_points, const void* points,
                                const void* points_size, void* dense, void* workspace, size_t workspace_bytes,
                                void* stream_, bool count_pairs, bool keep_status = false) {
    if (!bb || !points || !points_size || !workspace) return SESSD_ERR_NULL;
    if (bb->has_s2d && !dense) return SESSD_ERR_NULL;
    if (!voxel_params_ok(&bb->vp, batch, max_points)) return SESSD_ERR_PARAM;
    if ((uint64_t)batch * bb->max_voxels * 27ull > 0x7FFFFFFFull) return SESSD_ERR_PARAM;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    Bump bump(workspace);
    BackboneWorkspace w;
    backbone_layout(bump, bb, batch, max_points, &w);
    if (bump.total() > workspace_bytes) return SESSD_ERR_WORKSPACE;
    if (!workspace_aligned(workspace)) return SESSD_ERR_PARAM;
    const int maxV = bb->max_voxels;
    // keep_status (pipelines): word 0 is left alone, so that it collects the conditions of every group of a run
    SESSD_CUDA(cudaMemsetAsync(w.status + (keep_status ? 1 : 0), 0, (kStatusInts - (keep_status ? 1 : 0)) * sizeof(int32_t),
                               stream));
    // one launch resets everything the call needs: the voxeliser's table and the bucket table (0xFF), the grids and
    // tile masks (0), and the BEV map (0; by cudaMemsetAsync when its size is not a multiple of 16 bytes)
    FillRanges fills{};
    fills.ptr[0] = static_cast<uint4*>(w.ones_base), fills.n16[0] = w.ones_bytes / 16, fills.ones[0] = 1;
    fills.ptr[1] = static_cast<uint4*>(w.zero_base), fills.n16[1] = w.zero_bytes / 16, fills.ones[1] = 0;
    fills.ptr[2] = static_cast<uint4*>(static_cast<void*>(w.vox.table_base)), fills.n16[2] = w.vox.table_bytes / 16,
    fills.ones[2] = 1;
    const bool table_in_fill = w.vox.table_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(w.vox.table_base) % 16 == 0;
    if (!table_in_fill) fills.n16[2] = 0;
    if (bb->has_s2d) {
        const size_t bytes = (size_t)batch * bb->s2d.feature_map_channel * bb->s2d.feature_map_size_z *
                             (bb->s2d.feature_map_size_y + bb->pad.top + bb->pad.bottom) *
                             (bb->s2d.feature_map_size_x + bb->pad.left + bb->pad.right) * esize(bb->dtype);
        if (bytes % 16 == 0 && reinterpret_cast<uintptr_t>(dense) % 16 == 0)
            fills.ptr[3] = static_cast<uint4*>(dense), fills.n16[3] = bytes / 16, fills.ones[3] = 0;
        else
            SESSD_CUDA(cudaMemsetAsync(dense, 0, bytes, stream));
    }
    int rc = launch_fill_ranges(fills, stream);
    if (rc) return rc;
    rc = voxelize_run(&bb->vp, batch, max_points, bb->dtype, static_cast<const float*>(points),
                      static_cast<const int32_t*>(points_size), w.voxel_feat, w.coors[0], w.num[0], w.vox,
                      /*zero_tail=*/false, stream, table_in_fill);
    if (rc) return rc;
    std::vector<char> nbr_ready(bb->nlevels, 0);
    const void* cur = w.voxel_feat;
    for (size_t i = 0; i < bb->layers.size(); ++i) {
        const sessd_backbone::Layer& L = bb->layers[i];
        const int32_t* nbr;
        const uint32_t* tile_mask;
        if (L.p.subm) {
            if (!nbr_ready[L.level_in]) {
                if (L.level_in == 0) {
                    // the voxeliser's rows: x-grouped table, then one thread per row looks its 27 neighbours up
                    rc = launch_bucket_build(w.coors[0], w.num[0], batch, maxV, &bb->level_shape[0], w.buckets0, w.status,
                                             stream);
                    if (rc) return rc;
                    rc = launch_nbr_build_subm(w.coors[0], w.num[0], batch, maxV, L.g.in_shape, w.buckets0, w.nbr_subm[0],
                                               w.mask_subm[0], stream);
                } else {
                    rc = launch_map_rows(w.coors[L.level_in], w.num[L.level_in], batch, maxV, L.g, w.bits[L.level_in],
                                         w.nbr_subm[L.level_in], w.mask_subm[L.level_in], stream);
                }
                if (rc) return rc;
                nbr_ready[L.level_in] = 1;
            }
            nbr = w.nbr_subm[L.level_in];
            tile_mask = w.mask_subm[L.level_in];
        } else {
            rc = launch_mark_outputs(w.coors[L.level_in], w.num[L.level_in], batch, maxV, L.g, w.bits[L.level_out], stream);
            if (rc) return rc;
            rc = launch_number_outputs(w.bits[L.level_out], batch, maxV, w.chunk_counts, w.coors[L.level_out],
                                       w.num[L.level_out], w.status, stream);
            if (rc) return rc;
            if (L.level_in == 0)   // no grid for the voxeliser's rows: every candidate finds its output row instead
                rc = launch_scatter_rows(w.coors[0], w.num[0], w.num[L.level_out], batch, maxV, L.g, w.bits[L.level_out],
                                         w.nbr_strided, w.mask_layer[i], stream);
            else
                rc = launch_map_rows(w.coors[L.level_out], w.num[L.level_out], batch, maxV, L.g, w.bits[L.level_in],
                                     w.nbr_strided, w.mask_layer[i], stream);
            if (rc) return rc;
            nbr = w.nbr_strided;
            tile_mask = w.mask_layer[i];
        }
        if (count_pairs) {
            auto* counters = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(w.status) + 256);
            rc = launch_count_pairs(nbr, w.num[L.level_out], batch, maxV, L.g.kvol, counters + i, stream);
            if (rc) return rc;
        }
        ConvLaunch c{};
        c.in = cur;
        c.out = w.feat[i];
        c.nbr = nbr;
        c.tile_mask = tile_mask;
        c.out_num = w.num[L.level_out];
        c.weights = L.w->impl.w;
        c.umma_weights = L.w->impl.umma_w;
        c.scale = L.w->impl.scale;
        c.shift = L.w->impl.shift;
        c.relu = L.w->impl.relu;
        c.batch = batch;
        c.max_voxels = maxV;
        c.kvol = L.g.kvol;
        c.cin = L.p.in_channel;
        c.cout = L.p.out_channel;
        c.dtype = bb->dtype;
        c.status = w.status;
        c.debug_withhold_weights = L.w->impl.debug_withhold;
        c.scale_host = L.w->impl.host_scale;
        c.shift_host = L.w->impl.host_shift;
        if (bb->has_s2d && i + 1 == bb->layers.size()) {
            // The padded plane is (top + H + bottom) x (left + W + right); starting the scatter (top, left)
            // into it folds the reference's ZeroPad2dPlugin (zeroPad2d.cu:192-198) into this epilogue.
            c.D = bb->s2d.feature_map_size_z;
            c.H = bb->s2d.feature_map_size_y + bb->pad.top + bb->pad.bottom;
            c.W = bb->s2d.feature_map_size_x + bb->pad.left + bb->pad.right;
            c.dense = static_cast<char*>(dense) + ((size_t)bb->pad.top * c.W + bb->pad.left) * esize(bb->dtype);
            c.out_coors = w.coors[L.level_out];
        }
        rc = choose_conv(c, stream);
        if (rc) return rc;
        cur = w.feat[i];
    }
    return SESSD_OK;
}

int sessd_backbone_enqueue(const sessd_backbone* bb, int batch, int max_points, const void* points,
                           const void* points_size, void* dense, void* workspace, size_t workspace_bytes,
                           void* stream) {
    return backbone_enqueue_impl(bb, batch, max_points, points, points_size, dense, workspace, workspace_bytes, stream,
                                 false);
}

int sessd_backbone_pair_counts(const sessd_backbone* bb, int batch, int max_points, const void* points,
                               const void* points_size, void* dense, void* workspace, size_t workspace_bytes,
                               void* stream, int64_t* host_counts) {
    if (!host_counts) return SESSD_ERR_NULL;
    int rc = backbone_enqueue_impl(bb, batch, max_points, points, points_size, dense, workspace, workspace_bytes,
                                   stream, true);
    if (rc) return rc;
    SESSD_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    SESSD_CUDA(cudaMemcpy(host_counts, static_cast<char*>(workspace) + 256, sizeof(int64_t) * bb->layers.size(),
                          cudaMemcpyDeviceToHost));
    return SESSD_OK;
}

int sessd_backbone_layer_view(const sessd_backbone* bb, int batch, int max_points, void* workspace, int layer,
                              void** features, void** coors, void** voxel_num) {
    if (!bb || !workspace) return SESSD_ERR_NULL;
    if (!voxel_params_ok(&bb->vp, batch, max_points) || layer < -1 || layer >= (int)bb->layers.size()) return SESSD_ERR_PARAM;
    Bump bump(workspace);
    BackboneWorkspace w;
    backbone_layout(bump, bb, batch, max_points, &w);
    const int level = layer < 0 ? 0 : bb->layers[layer].level_out;
    if (features) *features = layer < 0 ? w.voxel_feat : w.feat[layer];
    if (coors) *coors = w.coors[level];
    if (voxel_num) *voxel_num = w.num[level];
    return SESSD_OK;
}

int sessd_backbone_final_level(const sessd_backbone* bb) { return bb ? bb->nlevels - 1 : SESSD_ERR_NULL; }

int sessd_backbone_set_padding(sessd_backbone* bb, const sessd_pad2d_params* pad) {
    if (!bb || !pad) return SESSD_ERR_NULL;
    if (!bb->has_s2d || !pad_ok(pad)) return SESSD_ERR_PARAM;
    bb->pad = *pad;
    return SESSD_OK;
}

}  // extern "C"

// ---- host-buffer pipeline ----------------------------------------------------------------------

struct sessd_pipeline {
    const sessd_backbone* bb;
    int batch, max_points, nstreams;
    size_t ws_bytes, dense_bytes;
    std::vector<cudaStream_t> streams;
    std::vector<void*> ws, dense, pts;
    std::vector<int32_t*> sizes;
    std::vector<cudaEvent_t> done;
    cudaEvent_t start;
    // Host-buffer runs: the points of a slot's next group are copied in (stream h2d) while its current group
    // computes, and a group's BEV maps are copied out (stream d2h) while the slot's next group computes. Each
    // slot therefore has two input and two BEV buffers, used alternately ([2 * s + half]; half 0 are the
    // buffers above, which every other kind of run uses alone).
    cudaStream_t h2d, d2h;
    cudaEvent_t bev_all;                                   // the output stream has copied the run's last BEV maps
    std::vector<void*> pts_alt, dense_alt;
    std::vector<int32_t*> sizes_alt;
    std::vector<cudaEvent_t> in_ready, in_free, bev_out;   // [2 * s + half]
    std::vector<int> last_half;                            // BEV buffer half of the slot's latest group
    // optional: the launch sequence of one full group, captured once per stream slot and replayed
    bool use_graphs;
    std::vector<cudaGraphExec_t> graphs;
    std::vector<char> warmed;   // slot has run one plain enqueue (kernels configured) before any capture
    std::vector<uint64_t> graph_kernels;   // kernels in the slot's graph, for the launch counter
};

extern "C" {

void sessd_pipeline_destroy(sessd_pipeline* pl) {
    if (!pl) return;
    for (auto s : pl->streams) if (s) cudaStreamSynchronize(s);
    for (auto p : pl->ws) if (p) cudaFree(p);
    for (auto p : pl->dense) if (p) cudaFree(p);
    for (auto p : pl->pts) if (p) cudaFree(p);
    for (auto p : pl->sizes) if (p) cudaFree(p);
    if (pl->h2d) cudaStreamSynchronize(pl->h2d);
    if (pl->d2h) cudaStreamSynchronize(pl->d2h);
    for (auto p : pl->pts_alt) if (p) cudaFree(p);
    for (auto p : pl->dense_alt) if (p) cudaFree(p);
    for (auto p : pl->sizes_alt) if (p) cudaFree(p);
    for (auto e : pl->in_ready) if (e) cudaEventDestroy(e);
    for (auto e : pl->in_free) if (e) cudaEventDestroy(e);
    for (auto e : pl->bev_out) if (e) cudaEventDestroy(e);
    if (pl->bev_all) cudaEventDestroy(pl->bev_all);
    if (pl->h2d) cudaStreamDestroy(pl->h2d);
    if (pl->d2h) cudaStreamDestroy(pl->d2h);
    for (auto g : pl->graphs) if (g) cudaGraphExecDestroy(g);
    for (auto e : pl->done) if (e) cudaEventDestroy(e);
    if (pl->start) cudaEventDestroy(pl->start);
    for (auto s : pl->streams) if (s) cudaStreamDestroy(s);
    delete pl;
}

int sessd_pipeline_create(const sessd_backbone* bb, int batch, int max_points, int nstreams, sessd_pipeline** out) {
    if (!bb || !out) return SESSD_ERR_NULL;
    if (nstreams < 1 || nstreams > 16) return SESSD_ERR_PARAM;
    const size_t ws_bytes = sessd_backbone_workspace_bytes(bb, batch, max_points);
    if (ws_bytes == 0) return SESSD_ERR_PARAM;
    auto* pl = new sessd_pipeline();
    pl->bb = bb;
    pl->batch = batch;
    pl->max_points = max_points;
    pl->nstreams = nstreams;
    pl->ws_bytes = ws_bytes;
    pl->start = nullptr;
    pl->dense_bytes = bb->has_s2d ? (size_t)batch * bb->s2d.feature_map_channel * bb->s2d.feature_map_size_z *
                                        (bb->s2d.feature_map_size_y + bb->pad.top + bb->pad.bottom) *
                                        (bb->s2d.feature_map_size_x + bb->pad.left + bb->pad.right) *
                                        (bb->dtype == SESSD_F32 ? 4 : 2)
                                  : 0;
    pl->streams.assign(nstreams, nullptr);
    pl->ws.assign(nstreams, nullptr);
    pl->dense.assign(nstreams, nullptr);
    pl->pts.assign(nstreams, nullptr);
    pl->sizes.assign(nstreams, nullptr);
    pl->done.assign(nstreams, nullptr);
    pl->use_graphs = false;
    pl->graphs.assign(nstreams, nullptr);
    pl->warmed.assign(nstreams, 0);
    pl->graph_kernels.assign(nstreams, 0);
    pl->h2d = pl->d2h = nullptr;
    pl->bev_all = nullptr;
    pl->pts_alt.assign(nstreams, nullptr);
    pl->dense_alt.assign(nstreams, nullptr);
    pl->sizes_alt.assign(nstreams, nullptr);
    pl->in_ready.assign(2 * nstreams, nullptr);
    pl->in_free.assign(2 * nstreams, nullptr);
    pl->bev_out.assign(2 * nstreams, nullptr);
    pl->last_half.assign(nstreams, 0);
    cudaError_t e = cudaEventCreate(&pl->start);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&pl->h2d, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&pl->d2h, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pl->bev_all, cudaEventDisableTiming);
    for (int i = 0; i < 2 * nstreams && e == cudaSuccess; ++i) {
        e = cudaEventCreateWithFlags(&pl->in_ready[i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pl->in_free[i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pl->bev_out[i], cudaEventDisableTiming);
    }
    for (int s = 0; s < nstreams && e == cudaSuccess; ++s) {
        e = cudaStreamCreateWithFlags(&pl->streams[s], cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaMalloc(&pl->ws[s], ws_bytes);
        if (e == cudaSuccess && pl->dense_bytes) e = cudaMalloc(&pl->dense[s], pl->dense_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&pl->pts[s], (size_t)batch * max_points * 16);
        if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&pl->sizes[s]), (size_t)batch * 4);
        if (e == cudaSuccess) e = cudaEventCreate(&pl->done[s]);
    }
    if (e != cudaSuccess) {
        set_cuda_error(e, "sessd_pipeline_create");
        sessd_pipeline_destroy(pl);
        return SESSD_ERR_CUDA;
    }
    *out = pl;
    return SESSD_OK;
}

int sessd_pipeline_use_graphs(sessd_pipeline* pl, int enable) {
    if (!pl) return SESSD_ERR_NULL;
    pl->use_graphs = enable != 0;
    return SESSD_OK;
}

void* sessd_pipeline_dense(sessd_pipeline* pl, int s) {
    if (!pl || s < 0 || s >= pl->nstreams) return nullptr;
    return pl->last_half[s] ? pl->dense_alt[s] : pl->dense[s];
}

void* sessd_pipeline_workspace(sessd_pipeline* pl, int s) {
    if (!pl || s < 0 || s >= pl->nstreams) return nullptr;
    return pl->ws[s];
}

static int pipeline_run(sessd_pipeline* pl, const void* points, const int32_t* sizes, int nframes, bool host,
                        int32_t* host_voxel_num, int32_t* host_status, float* elapsed_ms, void* host_dense = nullptr) {
    if (!pl || !points || !sizes) return SESSD_ERR_NULL;
    if (nframes < 1) return SESSD_ERR_PARAM;
    const sessd_backbone* bb = pl->bb;
    const size_t frame_bytes = (size_t)pl->max_points * 16;
    const int last_layer = (int)bb->layers.size() - 1;
    // Host-buffer runs without graph replay overlap the copies with the compute (see sessd_pipeline); the second
    // set of buffers is allocated on the first such run.
    const bool overlap = host && !pl->use_graphs;
    if (overlap) {
        for (int s = 0; s < pl->nstreams; ++s) {
            if (!pl->pts_alt[s]) SESSD_CUDA(cudaMalloc(&pl->pts_alt[s], (size_t)pl->batch * pl->max_points * 16));
            if (!pl->sizes_alt[s])
                SESSD_CUDA(cudaMalloc(reinterpret_cast<void**>(&pl->sizes_alt[s]), (size_t)pl->batch * 4));
            if (host_dense && pl->dense_bytes && !pl->dense_alt[s])
                SESSD_CUDA(cudaMalloc(&pl->dense_alt[s], pl->dense_bytes));
        }
    }
    SESSD_CUDA(cudaEventRecord(pl->start, pl->streams[0]));
    for (int s = 1; s < pl->nstreams; ++s) SESSD_CUDA(cudaStreamWaitEvent(pl->streams[s], pl->start, 0));
    if (overlap) SESSD_CUDA(cudaStreamWaitEvent(pl->h2d, pl->start, 0));
    // a slot's status word collects the conditions of all its groups of this run
    for (int s = 0; s < pl->nstreams; ++s) SESSD_CUDA(cudaMemsetAsync(pl->ws[s], 0, 4, pl->streams[s]));
    int group = 0;
    for (int f0 = 0; f0 < nframes; f0 += pl->batch, ++group) {
        const int s = group % pl->nstreams;
        const int nb = nframes - f0 < pl->batch ? nframes - f0 : pl->batch;
        cudaStream_t st = pl->streams[s];
        const void* dpts;
        const int32_t* dsizes;
        const int half = overlap ? (group / pl->nstreams) & 1 : 0;
        const int slot2 = 2 * s + half;
        void* dense_s = pl->dense[s];
        if (overlap) {
            // copy in on the input stream once the group that used this half before (two slot turns back) has run
            void* in_pts = half ? pl->pts_alt[s] : pl->pts[s];
            int32_t* in_sizes = half ? pl->sizes_alt[s] : pl->sizes[s];
            SESSD_CUDA(cudaStreamWaitEvent(pl->h2d, pl->in_free[slot2], 0));
            SESSD_CUDA(cudaMemcpyAsync(in_pts, static_cast<const char*>(points) + (size_t)f0 * frame_bytes,
                                       (size_t)nb * frame_bytes, cudaMemcpyHostToDevice, pl->h2d));
            SESSD_CUDA(cudaMemcpyAsync(in_sizes, sizes + f0, (size_t)nb * 4, cudaMemcpyHostToDevice, pl->h2d));
            SESSD_CUDA(cudaEventRecord(pl->in_ready[slot2], pl->h2d));
            SESSD_CUDA(cudaStreamWaitEvent(st, pl->in_ready[slot2], 0));
            dpts = in_pts;
            dsizes = in_sizes;
            if (host_dense && pl->dense_bytes) {
                // the BEV buffer of this half must have been copied out (its previous group's copy)
                if (half) dense_s = pl->dense_alt[s];
                SESSD_CUDA(cudaStreamWaitEvent(st, pl->bev_out[slot2], 0));
            }
        } else if (host) {
            SESSD_CUDA(cudaMemcpyAsync(pl->pts[s], static_cast<const char*>(points) + (size_t)f0 * frame_bytes,
                                       (size_t)nb * frame_bytes, cudaMemcpyHostToDevice, st));
            SESSD_CUDA(cudaMemcpyAsync(pl->sizes[s], sizes + f0, (size_t)nb * 4, cudaMemcpyHostToDevice, st));
            dpts = pl->pts[s];
            dsizes = pl->sizes[s];
        } else {
            dpts = static_cast<const char*>(points) + (size_t)f0 * frame_bytes;
            dsizes = sizes + f0;
        }
        int rc = SESSD_OK;
        // Graph path: only full groups, only outside per-launch profiling (events recorded inside a capture
        // cannot be timed), and only after the slot has run once plainly. The captured sequence reads the
        // slot's own staging buffers, so device-resident inputs are copied there first (device to device).
        if (pl->use_graphs && nb == pl->batch && !g_recorder && pl->warmed[s]) {
            if (!host) {
                SESSD_CUDA(cudaMemcpyAsync(pl->pts[s], dpts, (size_t)nb * frame_bytes, cudaMemcpyDeviceToDevice, st));
                SESSD_CUDA(cudaMemcpyAsync(pl->sizes[s], dsizes, (size_t)nb * 4, cudaMemcpyDeviceToDevice, st));
            }
            if (!pl->graphs[s]) {
                cudaGraph_t graph = nullptr;
                const uint64_t launches_before = g_launches.load(std::memory_order_relaxed);
                SESSD_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
                rc = backbone_enqueue_impl(bb, nb, pl->max_points, pl->pts[s], pl->sizes[s], pl->dense[s], pl->ws[s],
                                           pl->ws_bytes, st, false, true);
                const cudaError_t e_end = cudaStreamEndCapture(st, &graph);
                // the captured launches were recorded, not run: they count when the graph is launched
                pl->graph_kernels[s] = g_launches.load(std::memory_order_relaxed) - launches_before;
                g_launches.fetch_sub(pl->graph_kernels[s], std::memory_order_relaxed);
                if (rc) {
                    if (graph) cudaGraphDestroy(graph);
                    return rc;
                }
                if (e_end != cudaSuccess) {
                    set_cuda_error(e_end, "cudaStreamEndCapture");
                    return SESSD_ERR_CUDA;
                }
                const cudaError_t e_inst = cudaGraphInstantiate(&pl->graphs[s], graph, 0);
                cudaGraphDestroy(graph);
                if (e_inst != cudaSuccess) {
                    set_cuda_error(e_inst, "cudaGraphInstantiate");
                    return SESSD_ERR_CUDA;
                }
            }
            SESSD_CUDA(cudaGraphLaunch(pl->graphs[s], st));
            g_launches.fetch_add(pl->graph_kernels[s], std::memory_order_relaxed);
        } else {
            rc = backbone_enqueue_impl(bb, nb, pl->max_points, dpts, dsizes, dense_s, pl->ws[s], pl->ws_bytes, st, false,
                                       true);
            if (rc) return rc;
            if (nb == pl->batch) pl->warmed[s] = 1;
        }
        pl->last_half[s] = dense_s == pl->dense[s] ? 0 : 1;
        if (overlap) SESSD_CUDA(cudaEventRecord(pl->in_free[slot2], st));
        if (host && (host_voxel_num || host_status)) {
            void *feat, *coors, *num;
            rc = sessd_backbone_layer_view(bb, nb, pl->max_points, pl->ws[s], last_layer, &feat, &coors, &num);
            if (rc) return rc;
            if (host_voxel_num)
                SESSD_CUDA(cudaMemcpyAsync(host_voxel_num + f0, num, (size_t)nb * 4, cudaMemcpyDeviceToHost, st));
            if (host_status)
                SESSD_CUDA(cudaMemcpyAsync(host_status + f0, pl->ws[s], 4, cudaMemcpyDeviceToHost, st));
        }
        if (host && host_dense && pl->dense_bytes) {
            // the group's BEV maps go to the host region of its stream slot (a consumer takes them from there
            // before the slot's next group lands)
            const size_t per_frame = pl->dense_bytes / pl->batch;
            if (overlap) {
                // on the output stream, behind the group; the slot's stream goes on with its next group
                SESSD_CUDA(cudaEventRecord(pl->done[s], st));
                SESSD_CUDA(cudaStreamWaitEvent(pl->d2h, pl->done[s], 0));
                SESSD_CUDA(cudaMemcpyAsync(static_cast<char*>(host_dense) + (size_t)s * pl->dense_bytes, dense_s,
                                           (size_t)nb * per_frame, cudaMemcpyDeviceToHost, pl->d2h));
                SESSD_CUDA(cudaEventRecord(pl->bev_out[slot2], pl->d2h));
            } else {
                SESSD_CUDA(cudaMemcpyAsync(static_cast<char*>(host_dense) + (size_t)s * pl->dense_bytes, dense_s,
                                           (size_t)nb * per_frame, cudaMemcpyDeviceToHost, st));
            }
        }
    }
    if (overlap && host_dense && pl->dense_bytes) {
        // the run ends when the last BEV copies have landed: every slot's stream waits for the output stream
        SESSD_CUDA(cudaEventRecord(pl->bev_all, pl->d2h));
        for (int s = 0; s < pl->nstreams; ++s) SESSD_CUDA(cudaStreamWaitEvent(pl->streams[s], pl->bev_all, 0));
    }
    float worst = 0.f;
    for (int s = 0; s < pl->nstreams; ++s) SESSD_CUDA(cudaEventRecord(pl->done[s], pl->streams[s]));
    for (int s = 0; s < pl->nstreams; ++s) {
        SESSD_CUDA(cudaEventSynchronize(pl->done[s]));
        float t = 0.f;
        SESSD_CUDA(cudaEventElapsedTime(&t, pl->start, pl->done[s]));
        if (t > worst) worst = t;
    }
    if (host && host_status) {
        // the status word of a group was copied to the slot of its first frame: spread it
        for (int f0 = 0; f0 < nframes; f0 += pl->batch)
            for (int f = f0 + 1; f < nframes && f < f0 + pl->batch; ++f) host_status[f] = host_status[f0];
    }
    if (elapsed_ms) *elapsed_ms = worst;
    return SESSD_OK;
}

int sessd_pipeline_run_host(sessd_pipeline* pl, const float* host_points, const int32_t* host_sizes, int nframes,
                            int32_t* host_voxel_num, int32_t* host_status, float* elapsed_ms) {
    return pipeline_run(pl, host_points, host_sizes, nframes, true, host_voxel_num, host_status, elapsed_ms);
}

int sessd_pipeline_run_host_bev(sessd_pipeline* pl, const float* host_points, const int32_t* host_sizes, int nframes,
                                int32_t* host_voxel_num, int32_t* host_status, void* host_dense, float* elapsed_ms) {
    if (!host_dense) return SESSD_ERR_NULL;
    return pipeline_run(pl, host_points, host_sizes, nframes, true, host_voxel_num, host_status, elapsed_ms, host_dense);
}

int sessd_pipeline_run_device(sessd_pipeline* pl, const void* points, const void* sizes, int nframes,
                              float* elapsed_ms) {
    return pipeline_run(pl, points, static_cast<const int32_t*>(sizes), nframes, false, nullptr, nullptr, elapsed_ms);
}

}  // extern "C"
