// Host side of the C ABI (include/fmha_mxfp8_abi.h): the reference's generated host contract (validate / grid / launch),
// the shape dispatch and the one-call default path, over the sm_100a kernels of this directory.
#include "../../include/fmha_mxfp8_abi.h"
#include "kernels.h"

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace {

using b200mx::AttnParams;

static_assert(sizeof(fmha_mxfp8_attn_args) == 656, "vs128/t128 kernarg size");
static_assert(sizeof(fmha_mxfp8_kvsplit_args) == 648, "kvsplit kernarg size");
static_assert(sizeof(fmha_mxfp8_combine_args) == 36, "combine kernarg size");
#define OFFCHK(T, f, o) static_assert(offsetof(T, f) == (o), #T "." #f " offset")
OFFCHK(fmha_mxfp8_attn_args, ptr_o, 0x000); OFFCHK(fmha_mxfp8_attn_args, ptr_q, 0x010); OFFCHK(fmha_mxfp8_attn_args, ptr_k, 0x020);
OFFCHK(fmha_mxfp8_attn_args, ptr_v, 0x030); OFFCHK(fmha_mxfp8_attn_args, ext_ptr_peer_plan, 0x038); OFFCHK(fmha_mxfp8_attn_args, ext_ptr_lse, 0x040); OFFCHK(fmha_mxfp8_attn_args, ext_ptr_v_blockscale, 0x048);
OFFCHK(fmha_mxfp8_attn_args, ext_flags, 0x058); OFFCHK(fmha_mxfp8_attn_args, s_seq_len, 0x060); OFFCHK(fmha_mxfp8_attn_args, s_Seqs, 0x070);
OFFCHK(fmha_mxfp8_attn_args, s_Hs, 0x090); OFFCHK(fmha_mxfp8_attn_args, s_Bs, 0x0A0); OFFCHK(fmha_mxfp8_attn_args, s_gqa, 0x0B0);
OFFCHK(fmha_mxfp8_attn_args, s_k_Seqs, 0x0C0); OFFCHK(fmha_mxfp8_attn_args, s_k_Hs, 0x0D0); OFFCHK(fmha_mxfp8_attn_args, s_k_Bs, 0x0E0);
OFFCHK(fmha_mxfp8_attn_args, s_kv_seq_len, 0x110); OFFCHK(fmha_mxfp8_attn_args, s_q_head_num, 0x140); OFFCHK(fmha_mxfp8_attn_args, s_v_Seqs, 0x150);
OFFCHK(fmha_mxfp8_attn_args, s_v_Hs, 0x160); OFFCHK(fmha_mxfp8_attn_args, s_v_Bs, 0x170); OFFCHK(fmha_mxfp8_attn_args, s_o_Seqs, 0x180);
OFFCHK(fmha_mxfp8_attn_args, s_o_Hs, 0x190); OFFCHK(fmha_mxfp8_attn_args, s_o_Bs, 0x1A0); OFFCHK(fmha_mxfp8_attn_args, ptr_q_descale, 0x200);
OFFCHK(fmha_mxfp8_attn_args, ptr_k_descale, 0x210); OFFCHK(fmha_mxfp8_attn_args, ptr_v_descale, 0x220); OFFCHK(fmha_mxfp8_attn_args, s_descale_q_Bs, 0x230);
OFFCHK(fmha_mxfp8_attn_args, s_descale_q_Hs, 0x240); OFFCHK(fmha_mxfp8_attn_args, s_descale_k_Bs, 0x250); OFFCHK(fmha_mxfp8_attn_args, s_descale_k_Hs, 0x260);
OFFCHK(fmha_mxfp8_attn_args, abi_tail, 0x280);
OFFCHK(fmha_mxfp8_kvsplit_args, s_descale_k_Hs, 0x260); OFFCHK(fmha_mxfp8_kvsplit_args, ptr_ohat, 0x270); OFFCHK(fmha_mxfp8_kvsplit_args, ptr_lse, 0x278);
OFFCHK(fmha_mxfp8_kvsplit_args, kvs_splits, 0x280); OFFCHK(fmha_mxfp8_kvsplit_args, kvs_rows_total, 0x284);
OFFCHK(fmha_mxfp8_combine_args, ptr_ohat, 0x00); OFFCHK(fmha_mxfp8_combine_args, ptr_lse, 0x08); OFFCHK(fmha_mxfp8_combine_args, ptr_out, 0x10);
OFFCHK(fmha_mxfp8_combine_args, rows_total, 0x18); OFFCHK(fmha_mxfp8_combine_args, d, 0x1C); OFFCHK(fmha_mxfp8_combine_args, splits, 0x20);

const char* const kNames[4] = {"fmha_fwd_hd128_mxfp8_v3_vs128", "fmha_fwd_hd128_mxfp8_v3_t128", "fmha_fwd_hd128_mxfp8_v3_kvsplit",
                               "fmha_fwd_hd128_mxfp8_v3_kvsplit_combine8h"};
const char* const kClassNames[6] = {"", "GV-HOST-EXTENT", "GV-HOST-KA-RANGE", "GV-HOST-KA-IS", "GV-HOST-GRID", "GV-HOST-SYM"};

int fail(char* err, size_t cap, int cls, const char* msg) {
    if (err && cap) {
        if (cls >= 1 && cls <= 5) std::snprintf(err, cap, "%s: %s", kClassNames[cls], msg);
        else std::snprintf(err, cap, "%s", msg);
    }
    return cls;
}

// The u32 kernel argument at a byte offset (the reference's `ka(off)`).
int64_t ka(const void* args, uint32_t off) {
    uint32_t v;
    std::memcpy(&v, static_cast<const uint8_t*>(args) + off, 4);
    return static_cast<int64_t>(v);
}

constexpr int64_t kI64Max = 9223372036854775807LL;

int validate_attention(int kernel, const void* a, const fmha_mxfp8_buffer_sizes& sz, const uint32_t grid[3], const fmha_mxfp8_symbols& sy,
                       char* err, size_t cap) {
    const bool split = kernel == FMHA_MXFP8_KVSPLIT;
    char msg[160];
    // the batch count is the symbol B in the split contract and grid z in the unsplit ones
    const int64_t nb = split ? sy.B : static_cast<int64_t>(grid[2]);
    struct Ext { const char* name; uint64_t have; int64_t need; };
    const Ext ext[] = {
        {"ptr_q", sz.ptr_q, nb * ka(a, 0xA0)},
        {"ptr_k", sz.ptr_k, nb * ka(a, 0xE0)},
        {"ptr_v", sz.ptr_v, nb * ka(a, 0x170)},
        {"ptr_o", sz.ptr_o, nb * ka(a, 0x1A0)},
        {"ptr_q_descale", sz.ptr_q_descale, nb * ka(a, 0x230) + 2048LL * ka(a, 0x140)},
        {"ptr_k_descale", sz.ptr_k_descale, nb * ka(a, 0x250) + 2560LL * ka(a, 0x140)},
        {"ptr_v_descale", sz.ptr_v_descale, 4096LL},
        {"ptr_ohat", sz.ptr_ohat, split ? ka(a, 0x280) * ka(a, 0x284) * 512LL : 0LL},
        {"ptr_lse", sz.ptr_lse, split ? ka(a, 0x280) * ka(a, 0x284) * 4LL : 0LL},
    };
    for (const Ext& e : ext) {
        if (e.have < static_cast<uint64_t>(e.need)) {
            std::snprintf(msg, sizeof msg, "%s: buffer %s smaller than declared allocation", e.name, e.name);
            return fail(err, cap, FMHA_MXFP8_E_EXTENT, msg);
        }
    }
    struct Rng { uint32_t off; int64_t lo, hi; bool split_only; };
    const Rng rng[] = {
        {0xB0, 1, 16, false},   {0x60, 1, kI64Max, false}, {0x110, 1, kI64Max, false}, {0x90, 128, 128, false}, {0xD0, 128, 128, false},
        {0x160, 128, 128, false}, {0x190, 256, 256, false}, {0x240, 4, 4, false},        {0x260, 4, 4, false},    {0x280, 1, kI64Max, true},
        {0x284, 1, kI64Max, true},
    };
    for (const Rng& r : rng) {
        if (r.split_only && !split) continue;
        if (ka(a, r.off) < r.lo || ka(a, r.off) > r.hi) {
            std::snprintf(msg, sizeof msg, "ka(0x%X) outside contract", r.off);
            return fail(err, cap, FMHA_MXFP8_E_KA_RANGE, msg);
        }
    }
    struct Rel { uint32_t off; int64_t want; bool split_only; };
    const Rel rel[] = {
        {0x140, sy.HK * ka(a, 0xB0), false},
        {0x70, ka(a, 0x140) * 128LL, false},
        {0xA0, ka(a, 0x60) * ka(a, 0x70), false},
        {0xC0, sy.HK * 128LL, false},
        {0xE0, ka(a, 0x110) * ka(a, 0xC0), false},
        {0x150, ka(a, 0xC0), false},
        {0x170, ka(a, 0xE0), false},
        {0x180, ka(a, 0x140) * 256LL, false},
        {0x1A0, ka(a, 0x60) * ka(a, 0x180), false},
        {0x230, ka(a, 0x60) * (ka(a, 0x140) * 4LL), false},
        {0x250, ka(a, 0x110) * (sy.HK * 4LL), false},
        {0x284, (sy.B * ka(a, 0x60)) * ka(a, 0x140), true},
    };
    for (const Rel& r : rel) {
        if (r.split_only && !split) continue;
        if (ka(a, r.off) != r.want) {
            std::snprintf(msg, sizeof msg, "ka(0x%X) relation failed", r.off);
            return fail(err, cap, FMHA_MXFP8_E_KA_IS, msg);
        }
    }
    const int64_t rows = kernel == FMHA_MXFP8_T128 ? 128 : 256;
    if (static_cast<int64_t>(grid[1]) != ka(a, 0x140)) return fail(err, cap, FMHA_MXFP8_E_GRID, "grid axis 1 relation failed");
    if (static_cast<int64_t>(grid[0]) != (ka(a, 0x60) + rows - 1) / rows) return fail(err, cap, FMHA_MXFP8_E_GRID, "grid axis 0 relation failed");
    if (split) {
        if (static_cast<int64_t>(grid[2]) != sy.B * ka(a, 0x280)) return fail(err, cap, FMHA_MXFP8_E_GRID, "grid axis 2 relation failed");
        if (sy.KL < 0) return fail(err, cap, FMHA_MXFP8_E_SYM, "symbol KL outside contract");
    }
    return FMHA_MXFP8_OK;
}

int validate_combine(const void* a, const fmha_mxfp8_buffer_sizes& sz, char* err, size_t cap) {
    const int64_t rows = ka(a, 0x18), d = ka(a, 0x1C), splits = ka(a, 0x20);
    if (sz.ptr_ohat < static_cast<uint64_t>(splits * rows * 512LL)) return fail(err, cap, FMHA_MXFP8_E_EXTENT, "ptr_ohat: buffer ptr_ohat smaller than declared allocation");
    if (sz.ptr_lse < static_cast<uint64_t>(splits * rows * 4LL)) return fail(err, cap, FMHA_MXFP8_E_EXTENT, "ptr_lse: buffer ptr_lse smaller than declared allocation");
    if (sz.ptr_out < static_cast<uint64_t>(rows * 256LL)) return fail(err, cap, FMHA_MXFP8_E_EXTENT, "ptr_out: buffer ptr_out smaller than declared allocation");
    if (rows < 1) return fail(err, cap, FMHA_MXFP8_E_KA_RANGE, "ka(0x18) outside contract");
    if (d != 128) return fail(err, cap, FMHA_MXFP8_E_KA_RANGE, "ka(0x1C) outside contract");
    if (splits < 1) return fail(err, cap, FMHA_MXFP8_E_KA_RANGE, "ka(0x20) outside contract");
    return FMHA_MXFP8_OK;
}

// ---- TMA descriptors -------------------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    });
    return fn;
}

// A [batch, seq, heads, 128] e4m3 tensor as a 4-D map (head dim, head, row, batch) with a box of `box_rows` rows x 128 bytes, 128-byte
// swizzle. Rows past `seq` read as zero.
int make_tile_map(CUtensorMap* m, const void* base, uint64_t seq, uint64_t heads, uint64_t batches, uint64_t head_stride, uint64_t row_stride,
                  uint64_t batch_stride, uint32_t box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return -static_cast<int>(cudaErrorSymbolNotFound);
    const cuuint64_t dims[4] = {128, heads, seq, batches};
    const cuuint64_t strides[3] = {head_stride, row_stride, batch_stride == 0 ? row_stride * seq : batch_stride};
    const cuuint32_t box[4] = {128, 1, box_rows, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r);
}

// The bf16 output [batch, seq, heads, 128] as a 4-D map (head dim, head, row, batch) with a 128-row x 64-column box, 128-byte swizzle:
// the shape of one warpgroup's TMA store. Rows past `seq` are not written.
int make_out_map(CUtensorMap* m, void* base, uint64_t seq, uint64_t heads, uint64_t batches, uint64_t head_stride, uint64_t row_stride,
                 uint64_t batch_stride) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return -static_cast<int>(cudaErrorSymbolNotFound);
    const cuuint64_t dims[4] = {128, heads, seq, batches};
    const cuuint64_t strides[3] = {head_stride, row_stride, batch_stride == 0 ? row_stride * seq : batch_stride};
    const cuuint32_t box[4] = {64, 1, 128, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r);
}

// The split kernel's partials [splits][B*S*H rows][128] as a 5-D map (head dim, head, row, batch, split), 128-byte swizzle: f16 rows of
// 256 bytes with a 128-row x 64-column box, or f32 rows of 512 bytes with a 128-row x 32-column box (either box is 128 bytes wide).
int make_partial_map(CUtensorMap* m, void* base, uint64_t seq, uint64_t heads, uint64_t batches, uint64_t splits, bool f32) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return -static_cast<int>(cudaErrorSymbolNotFound);
    const uint64_t rb = f32 ? 512 : 256;
    const cuuint64_t dims[5] = {128, heads, seq, batches, splits};
    const cuuint64_t strides[4] = {rb, heads * rb, seq * heads * rb, batches * seq * heads * rb};
    const cuuint32_t box[5] = {f32 ? 32u : 64u, 1, 128, 1, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUresult r = enc(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r);
}

uint32_t log2_u32(uint32_t x) {
    uint32_t l = 0;
    while ((1u << l) < x) ++l;
    return l;
}

std::atomic<float*> g_trace{nullptr};

int launch_attention_kernel(int kernel, const void* args, const uint32_t grid[3], cudaStream_t stream) {
    // the common prefix of the three attention argument blocks
    const fmha_mxfp8_attn_args* a = static_cast<const fmha_mxfp8_attn_args*>(args);
    const bool split = kernel == FMHA_MXFP8_KVSPLIT;
    AttnParams p{};
    p.S = a->s_seq_len;
    p.SK = a->s_kv_seq_len;
    p.H = a->s_q_head_num;
    if (a->s_gqa == 0 || p.H == 0 || p.S == 0 || p.SK == 0) return FMHA_MXFP8_E_KA_RANGE;
    // the kernels find a head's KV head with a shift (crates/amdgpu-stage/src/components.rs:8-17): the group size must be a power of two that divides H
    if ((a->s_gqa & (a->s_gqa - 1u)) != 0u || p.H % a->s_gqa != 0u) return FMHA_MXFP8_E_KA_RANGE;
    p.HK = p.H / a->s_gqa;
    p.gqa_shift = log2_u32(a->s_gqa);
    p.o = static_cast<uint8_t*>(a->ptr_o);
    p.o_row_stride = a->s_o_Seqs;
    p.o_batch_stride = a->s_o_Bs;
    p.q_descale = static_cast<const uint8_t*>(a->ptr_q_descale);
    p.k_descale = static_cast<const uint8_t*>(a->ptr_k_descale);
    p.v_descale = static_cast<const float*>(a->ptr_v_descale);
    p.qs_batch_stride = a->s_descale_q_Bs;
    p.ks_batch_stride = a->s_descale_k_Bs;
    p.flags = a->ext_flags;
    // V block scales (extension): a pointer is needed, and the mask and the diagnostics have no variant with them
    if ((p.flags & FMHA_MXFP8_FLAG_V_BLOCKSCALE) && (a->ext_ptr_v_blockscale == nullptr || (p.flags & FMHA_MXFP8_FLAG_CAUSAL) || g_trace.load(std::memory_order_relaxed) != nullptr))
        return FMHA_MXFP8_E_ARG;
    if ((p.flags & FMHA_MXFP8_FLAG_CAUSAL) && (split || p.SK < p.S)) return FMHA_MXFP8_E_ARG;   // causal: unsplit kernels, SK >= S
    p.v_blockscale = (p.flags & FMHA_MXFP8_FLAG_V_BLOCKSCALE) ? static_cast<const uint8_t*>(a->ext_ptr_v_blockscale) : nullptr;
    p.lse_nat = split ? nullptr : static_cast<float*>(a->ext_ptr_lse);
    p.trace = g_trace.load(std::memory_order_relaxed);
    p.status = b200mx::device_status_word();
    if (p.status == nullptr) return -static_cast<int>(cudaErrorInvalidSymbol);
    uint32_t B = grid[2];
    p.splits = 1;
    if (split) {
        const fmha_mxfp8_kvsplit_args* s = static_cast<const fmha_mxfp8_kvsplit_args*>(args);
        p.splits = s->kvs_splits;
        if (p.splits == 0 || (p.splits & (p.splits - 1)) != 0 || grid[2] % p.splits != 0) return FMHA_MXFP8_E_KA_RANGE;
        // every split must own a key tile (tests/gpu/ref_host.cpp:117-120)
        const uint32_t ntiles = (p.SK + 127) / 128, tps = (ntiles + p.splits - 1) / p.splits;
        if (static_cast<uint64_t>(p.splits - 1) * tps >= ntiles) return FMHA_MXFP8_E_KA_RANGE;
        p.split_log2 = log2_u32(p.splits);
        p.rows_total = s->kvs_rows_total;
        p.ohat = s->ptr_ohat;
        // the partial rows go to the GPUs that combine them (extension): one batch element; the plan was built for f16 or f32 partials and the launch must use the same
        p.peer = static_cast<const b200mx::PeerPlan*>(a->ext_ptr_peer_plan);
        if (p.peer != nullptr && (grid[2] != s->kvs_splits || s->kvs_splits != 1u)) return FMHA_MXFP8_E_ARG;
        p.lse2 = static_cast<float*>(s->ptr_lse);
        B = grid[2] / p.splits;
        // the fused merge (extension): counters, the final output, f16 partials that stay on this GPU
        if (p.flags & FMHA_MXFP8_FLAG_FUSED_COMBINE) {
            p.fused_counters = static_cast<uint32_t*>(s->ext_ptr_fused_counters);
            if (p.fused_counters == nullptr || (reinterpret_cast<uintptr_t>(p.fused_counters) & 3u) || p.o == nullptr || p.peer != nullptr ||
                (p.flags & FMHA_MXFP8_FLAG_F32_PARTIALS) || p.splits > 8u || g_trace.load(std::memory_order_relaxed) != nullptr)
                return FMHA_MXFP8_E_ARG;
        }
    }
    if (split && static_cast<uint64_t>(p.rows_total) != static_cast<uint64_t>(B) * p.S * p.H) return FMHA_MXFP8_E_KA_IS;
    // The four tensor maps depend on nothing but the argument block (pointers, extents, strides, flags): a call with the bytes of an
    // earlier one reuses its maps instead of encoding them again (four driver calls; a framework calls a layer with the same buffers
    // step after step). A few entries, replaced in turn; the lock is held for two short copies.
    struct MapSet {
        bool valid;
        int kernel;
        uint32_t grid_z;
        unsigned char args[sizeof(fmha_mxfp8_attn_args) > sizeof(fmha_mxfp8_kvsplit_args) ? sizeof(fmha_mxfp8_attn_args) : sizeof(fmha_mxfp8_kvsplit_args)];
        CUtensorMap tq, tk, tv, to;
    };
    constexpr int kMapSets = 8;
    static MapSet sets[kMapSets];
    static int next_set = 0;
    static std::mutex sets_lock;
    const size_t arg_bytes = split ? sizeof(fmha_mxfp8_kvsplit_args) : sizeof(fmha_mxfp8_attn_args);
    CUtensorMap tq, tk, tv, to;   // to: the output of the kernel's TMA stores: bf16 O, or the split kernel's partials
    bool have = false;
    {
        std::lock_guard<std::mutex> g(sets_lock);
        for (int i = 0; i < kMapSets && !have; ++i) {
            const MapSet& m = sets[i];
            if (m.valid && m.kernel == kernel && m.grid_z == grid[2] && std::memcmp(m.args, args, arg_bytes) == 0) {
                tq = m.tq; tk = m.tk; tv = m.tv; to = m.to;
                have = true;
            }
        }
    }
    if (!have) {
        int r = make_tile_map(&tq, a->ptr_q, p.S, p.H, B, a->s_Hs, a->s_Seqs, a->s_Bs, 128u);
        if (r) return r;
        r = make_tile_map(&tk, a->ptr_k, p.SK, p.HK, B, a->s_k_Hs, a->s_k_Seqs, a->s_k_Bs, b200mx::kKeysPerTile);
        if (r) return r;
        r = make_tile_map(&tv, a->ptr_v, p.SK, p.HK, B, a->s_v_Hs, a->s_v_Seqs, a->s_v_Bs, b200mx::kKeysPerTile);
        if (r) return r;
        if (!split) r = make_out_map(&to, a->ptr_o, p.S, p.H, B, a->s_o_Hs, a->s_o_Seqs, a->s_o_Bs);
        else r = make_partial_map(&to, p.ohat, p.S, p.H, B, p.splits, (p.flags & FMHA_MXFP8_FLAG_F32_PARTIALS) != 0u);
        if (r) return r;
        std::lock_guard<std::mutex> g(sets_lock);
        MapSet& m = sets[next_set];
        next_set = (next_set + 1) % kMapSets;
        m.valid = true;
        m.kernel = kernel;
        m.grid_z = grid[2];
        std::memcpy(m.args, args, arg_bytes);
        m.tq = tq; m.tk = tk; m.tv = tv; m.to = to;
    }
    const cudaError_t e = b200mx::launch_attention(tq, tk, tv, to, p, B, split, kernel == FMHA_MXFP8_T128 ? 128u : 256u, stream);
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

}  // namespace

namespace b200mx {
int encode_partial_map(CUtensorMap* m, void* base, uint64_t seq, uint64_t heads, uint64_t batches, uint64_t splits, bool f32) {
    return make_partial_map(m, base, seq, heads, batches, splits, f32);
}
__device__ uint32_t g_status_word = 0;
uint32_t* device_status_word() {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    return static_cast<uint32_t*>(p);
}
}  // namespace b200mx

extern "C" {

const char* fmha_mxfp8_kernel_name(int kernel) { return (kernel >= 0 && kernel < 4) ? kNames[kernel] : nullptr; }

size_t fmha_mxfp8_kernarg_size(int kernel) {
    switch (kernel) {
        case FMHA_MXFP8_VS128: case FMHA_MXFP8_T128: return sizeof(fmha_mxfp8_attn_args);
        case FMHA_MXFP8_KVSPLIT: return sizeof(fmha_mxfp8_kvsplit_args);
        case FMHA_MXFP8_COMBINE8H: return sizeof(fmha_mxfp8_combine_args);
        default: return 0;
    }
}

unsigned fmha_mxfp8_workgroup_size(int kernel) {
    switch (kernel) {
        case FMHA_MXFP8_VS128: case FMHA_MXFP8_KVSPLIT: return 512;
        case FMHA_MXFP8_T128: case FMHA_MXFP8_COMBINE8H: return 256;
        default: return 0;
    }
}

int fmha_mxfp8_validate(int kernel, const void* args, const fmha_mxfp8_buffer_sizes* sizes, const uint32_t grid[3],
                        const fmha_mxfp8_symbols* syms, char* err, size_t cap) {
    if (err && cap) err[0] = 0;
    if (!args || !sizes || kernel < 0 || kernel > 3) return fail(err, cap, FMHA_MXFP8_E_ARG, "bad kernel id or null argument");
    if (kernel == FMHA_MXFP8_COMBINE8H) return validate_combine(args, *sizes, err, cap);
    if (!grid || !syms) return fail(err, cap, FMHA_MXFP8_E_ARG, "grid and symbols are required");
    return validate_attention(kernel, args, *sizes, grid, *syms, err, cap);
}

int fmha_mxfp8_grid(int kernel, const void* args, const fmha_mxfp8_symbols* syms, uint32_t grid[3]) {
    if (!args || !grid || kernel < 0 || kernel > 3) return FMHA_MXFP8_E_ARG;
    if (kernel == FMHA_MXFP8_COMBINE8H) {
        const uint64_t n = static_cast<uint64_t>(ka(args, 0x18)) * 128u;
        uint64_t g = (n + 2047u) / 2048u;
        grid[0] = static_cast<uint32_t>(g < 1 ? 1 : g); grid[1] = 1; grid[2] = 1;
        return 0;
    }
    if (!syms) return FMHA_MXFP8_E_ARG;
    const int64_t rows = kernel == FMHA_MXFP8_T128 ? 128 : 256;
    grid[0] = static_cast<uint32_t>((ka(args, 0x60) + rows - 1) / rows);
    grid[1] = static_cast<uint32_t>(ka(args, 0x140));
    grid[2] = static_cast<uint32_t>(kernel == FMHA_MXFP8_KVSPLIT ? syms->B * ka(args, 0x280) : syms->B);
    return 0;
}

int fmha_mxfp8_launch(int kernel, const void* args, const uint32_t grid[3], void* stream) {
    if (!args || kernel < 0 || kernel > 3) return FMHA_MXFP8_E_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (kernel == FMHA_MXFP8_COMBINE8H) {
        const fmha_mxfp8_combine_args* c = static_cast<const fmha_mxfp8_combine_args*>(args);
        if (c->d != 128 || c->rows_total == 0 || c->splits == 0) return FMHA_MXFP8_E_KA_RANGE;
        // half-precision partials, as the reference's combine8h reads them (crates/amdgpu-kernels/src/fmha/io.rs:161-185)
        const cudaError_t e = b200mx::launch_combine(c->ptr_ohat, false, static_cast<const float*>(c->ptr_lse), static_cast<uint8_t*>(c->ptr_out), c->rows_total,
                                                     c->splits, st);
        return e == cudaSuccess ? 0 : -static_cast<int>(e);
    }
    if (!grid) return FMHA_MXFP8_E_ARG;
    return launch_attention_kernel(kernel, args, grid, st);
}

void fmha_mxfp8_dispatch(uint64_t b, uint64_t h, uint64_t s, uint64_t sk, int* path, uint32_t* splits) {
    const uint64_t blocks256 = ((s + 255) / 256) * h * b;
    const uint64_t ntiles = (sk + 127) / 128;
    uint64_t sp = 0;
    if (ntiles >= 16 && blocks256 <= 64) sp = 4;
    else if (ntiles >= 32 && blocks256 <= 128) sp = 2;
    if (sp > 0) {
        const uint64_t tps = (ntiles + sp - 1) / sp;
        if ((sp - 1) * tps < ntiles) {
            if (path) *path = FMHA_MXFP8_KVSPLIT;
            if (splits) *splits = static_cast<uint32_t>(sp);
            return;
        }
    }
    if (path) *path = blocks256 <= 64 ? FMHA_MXFP8_T128 : FMHA_MXFP8_VS128;
    if (splits) *splits = 0;
}

int fmha_mxfp8_auto(const fmha_mxfp8_problem* pr, int path, uint32_t splits, void* stream, int* path_out, uint32_t* splits_out,
                    char* err, size_t cap) {
    if (err && cap) err[0] = 0;
    if (!pr) return fail(err, cap, FMHA_MXFP8_E_ARG, "null problem");
    if (pr->HK == 0 || pr->H % pr->HK != 0) return fail(err, cap, FMHA_MXFP8_E_ARG, "H must be a multiple of HK");
    const uint32_t gqa = pr->H / pr->HK;
    if ((gqa & (gqa - 1)) != 0 || gqa > 16) return fail(err, cap, FMHA_MXFP8_E_ARG, "H / HK must be a power of two <= 16");
    if (path < 0) {
        fmha_mxfp8_dispatch(pr->B, pr->H, pr->S, pr->SK, &path, &splits);
        if ((pr->flags & FMHA_MXFP8_FLAG_CAUSAL) && path == FMHA_MXFP8_KVSPLIT) {   // the causal extension has no split form
            path = FMHA_MXFP8_VS128;
            splits = 0;
        }
    } else if (path == FMHA_MXFP8_KVSPLIT) {
        if (splits == 0) splits = 4;
        if (splits != 2 && splits != 4 && splits != 8) return fail(err, cap, FMHA_MXFP8_E_ARG, "splits must be 2, 4 or 8");
    } else if (path == FMHA_MXFP8_VS128 || path == FMHA_MXFP8_T128) {
        splits = 0;
    } else {
        return fail(err, cap, FMHA_MXFP8_E_ARG, "unknown path");
    }
    if (path_out) *path_out = path;
    if (splits_out) *splits_out = splits;

    const uint64_t S = pr->S, SK = pr->SK, H = pr->H, HK = pr->HK, B = pr->B;
    fmha_mxfp8_kvsplit_args a;   // a superset of the unsplit block up to 0x26F
    std::memset(&a, 0, sizeof a);
    a.ptr_o = pr->out; a.ptr_q = const_cast<void*>(pr->q); a.ptr_k = const_cast<void*>(pr->k); a.ptr_v = const_cast<void*>(pr->v);
    a.s_seq_len = pr->S; a.s_Seqs = static_cast<uint32_t>(H * 128); a.s_Hs = 128; a.s_Bs = static_cast<uint32_t>(S * H * 128);
    a.s_gqa = gqa; a.s_k_Seqs = static_cast<uint32_t>(HK * 128); a.s_k_Hs = 128; a.s_k_Bs = static_cast<uint32_t>(SK * HK * 128);
    a.s_kv_seq_len = pr->SK; a.s_q_head_num = pr->H;
    a.s_v_Seqs = a.s_k_Seqs; a.s_v_Hs = 128; a.s_v_Bs = a.s_k_Bs;
    a.s_o_Seqs = static_cast<uint32_t>(H * 256); a.s_o_Hs = 256; a.s_o_Bs = static_cast<uint32_t>(S * H * 256);
    a.ptr_q_descale = const_cast<void*>(pr->q_descale); a.ptr_k_descale = const_cast<void*>(pr->k_descale); a.ptr_v_descale = const_cast<void*>(pr->v_descale);
    a.s_descale_q_Bs = static_cast<uint32_t>(S * H * 4); a.s_descale_q_Hs = 4;
    a.s_descale_k_Bs = static_cast<uint32_t>(SK * HK * 4); a.s_descale_k_Hs = 4;
    a.ext_flags = (pr->flags & ~FMHA_MXFP8_FLAG_FUSED_COMBINE) | (pr->v_blockscale ? FMHA_MXFP8_FLAG_V_BLOCKSCALE : 0u);
    a.ext_ptr_v_blockscale = const_cast<void*>(pr->v_blockscale);
    if (S * H * 256 * 1ull > 0xFFFFFFFFull || SK * HK * 128 > 0xFFFFFFFFull) return fail(err, cap, FMHA_MXFP8_E_ARG, "a batch stride does not fit the u32 kernel argument");

    fmha_mxfp8_buffer_sizes sz;
    std::memset(&sz, 0, sizeof sz);
    sz.ptr_q = B * S * H * 128; sz.ptr_k = B * SK * HK * 128; sz.ptr_v = sz.ptr_k; sz.ptr_o = B * S * H * 256;
    sz.ptr_q_descale = pr->q_descale_bytes; sz.ptr_k_descale = pr->k_descale_bytes; sz.ptr_v_descale = pr->v_descale_bytes;
    fmha_mxfp8_symbols sy{static_cast<int64_t>(B), static_cast<int64_t>(HK), 0};

    if (path != FMHA_MXFP8_KVSPLIT) {
        fmha_mxfp8_attn_args u;
        std::memset(&u, 0, sizeof u);
        std::memcpy(&u, &a, offsetof(fmha_mxfp8_kvsplit_args, ptr_ohat));
        const uint32_t rows = path == FMHA_MXFP8_T128 ? 128 : 256;
        const uint32_t grid[3] = {static_cast<uint32_t>((S + rows - 1) / rows), pr->H, pr->B};
        int r = fmha_mxfp8_validate(path, &u, &sz, grid, &sy, err, cap);
        if (r) return r;
        r = fmha_mxfp8_launch(path, &u, grid, stream);
        if (r) return fail(err, cap, r, "launch failed");
        return 0;
    }
    const uint64_t rows_total = B * S * H;
    a.ptr_ohat = pr->ws_ohat; a.ptr_lse = pr->ws_lse; a.kvs_splits = splits; a.kvs_rows_total = static_cast<uint32_t>(rows_total);
    sz.ptr_ohat = pr->ws_ohat_bytes; sz.ptr_lse = pr->ws_lse_bytes;
    const uint32_t grid[3] = {static_cast<uint32_t>((S + 255) / 256), pr->H, pr->B * splits};
    int r = fmha_mxfp8_validate(FMHA_MXFP8_KVSPLIT, &a, &sz, grid, &sy, err, cap);
    if (r) return r;
    fmha_mxfp8_combine_args c;
    std::memset(&c, 0, sizeof c);
    c.ptr_ohat = pr->ws_ohat; c.ptr_lse = pr->ws_lse; c.ptr_out = pr->out;
    c.rows_total = static_cast<uint32_t>(rows_total); c.d = 128; c.splits = splits;
    fmha_mxfp8_buffer_sizes csz;
    std::memset(&csz, 0, sizeof csz);
    csz.ptr_ohat = pr->ws_ohat_bytes; csz.ptr_lse = pr->ws_lse_bytes; csz.ptr_out = sz.ptr_o;
    uint32_t cgrid[3];
    fmha_mxfp8_grid(FMHA_MXFP8_COMBINE8H, &c, nullptr, cgrid);
    r = fmha_mxfp8_validate(FMHA_MXFP8_COMBINE8H, &c, &csz, cgrid, nullptr, err, cap);
    if (r) return r;
    if (pr->flags & FMHA_MXFP8_FLAG_FUSED_COMBINE) {
        // one kernel: the counters sit behind the f16 partials in the f32-sized allocation and are cleared in front of every call
        const uint64_t n_blocks = B * H * ((S + 127) / 128), off = static_cast<uint64_t>(splits) * rows_total * 256u;
        if (off + n_blocks * 4u > pr->ws_ohat_bytes) return fail(err, cap, FMHA_MXFP8_E_ARG, "ws_ohat too small for the fused merge's counters");
        a.ext_flags |= FMHA_MXFP8_FLAG_FUSED_COMBINE;
        a.ext_ptr_fused_counters = static_cast<uint8_t*>(pr->ws_ohat) + off;
        const cudaError_t e = cudaMemsetAsync(a.ext_ptr_fused_counters, 0, n_blocks * 4u, static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return fail(err, cap, -static_cast<int>(e), "clearing the counters failed");
        r = fmha_mxfp8_launch(FMHA_MXFP8_KVSPLIT, &a, grid, stream);
        if (r) return fail(err, cap, r, "kvsplit launch failed");
        return 0;
    }
    r = fmha_mxfp8_launch(FMHA_MXFP8_KVSPLIT, &a, grid, stream);
    if (r) return fail(err, cap, r, "kvsplit launch failed");
    r = fmha_mxfp8_launch(FMHA_MXFP8_COMBINE8H, &c, cgrid, stream);
    if (r) return fail(err, cap, r, "combine launch failed");
    return 0;
}

int fmha_mxfp8_combine_f32(const void* ohat, const void* lse, void* out, uint32_t rows_total, uint32_t splits, void* stream) {
    if (!ohat || !lse || !out || rows_total == 0 || splits == 0) return FMHA_MXFP8_E_ARG;
    if ((reinterpret_cast<uintptr_t>(ohat) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u) || (reinterpret_cast<uintptr_t>(lse) & 3u)) return FMHA_MXFP8_E_ARG;
    const cudaError_t e = b200mx::launch_combine(ohat, true, static_cast<const float*>(lse), static_cast<uint8_t*>(out), rows_total, splits, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

int fmha_mxfp8_quantize_qk(const void* x_bf16, uint64_t rows, float mul, void* out_e4m3, void* out_scales, void* stream) {
    if (!x_bf16 || !out_e4m3 || !out_scales) return FMHA_MXFP8_E_ARG;
    if (rows == 0) return 0;
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) || (reinterpret_cast<uintptr_t>(out_e4m3) & 7u) || (reinterpret_cast<uintptr_t>(out_scales) & 3u)) return FMHA_MXFP8_E_ARG;
    const cudaError_t e = b200mx::launch_quantize_qk(x_bf16, rows, mul, out_e4m3, out_scales, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

int fmha_mxfp8_quantize_v(const void* x_bf16, uint64_t n_elems, void* out_e4m3, void* v_descale, void* stream) {
    if (!x_bf16 || !out_e4m3 || !v_descale || (n_elems & 7u)) return FMHA_MXFP8_E_ARG;
    if (n_elems == 0) return 0;
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) || (reinterpret_cast<uintptr_t>(out_e4m3) & 7u) || (reinterpret_cast<uintptr_t>(v_descale) & 7u)) return FMHA_MXFP8_E_ARG;
    const cudaError_t e = b200mx::launch_quantize_v(x_bf16, n_elems, out_e4m3, static_cast<float*>(v_descale), static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

int fmha_mxfp8_device_status(uint32_t* status) {
    uint32_t* d = b200mx::device_status_word();
    if (!d || !status) return FMHA_MXFP8_E_ARG;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return -static_cast<int>(e);
    e = cudaMemcpy(status, d, 4, cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

int fmha_mxfp8_trace_attach(void* dev_buf, size_t bytes) {
    if (dev_buf && bytes < FMHA_MXFP8_TRACE_BYTES) return FMHA_MXFP8_E_EXTENT;
    g_trace.store(static_cast<float*>(dev_buf), std::memory_order_relaxed);
    return 0;
}

int fmha_mxfp8_mma_issue_ceiling(int iters, int ctas, void* stream, float* ms) {
    if (iters < 2 || ctas < 1 || !ms) return FMHA_MXFP8_E_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint32_t* status = b200mx::device_status_word();
    if (!status) return -static_cast<int>(cudaErrorInvalidSymbol);
    cudaEvent_t e0, e1;
    cudaError_t e = cudaEventCreate(&e0);
    if (e != cudaSuccess) return -static_cast<int>(e);
    e = cudaEventCreate(&e1);
    if (e != cudaSuccess) { cudaEventDestroy(e0); return -static_cast<int>(e); }
    e = b200mx::launch_mma_issue_ceiling(8, ctas, status, st);   // warm-up
    if (e == cudaSuccess) e = cudaEventRecord(e0, st);
    if (e == cudaSuccess) e = b200mx::launch_mma_issue_ceiling(iters, ctas, status, st);
    if (e == cudaSuccess) e = cudaEventRecord(e1, st);
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    if (e == cudaSuccess) e = cudaEventElapsedTime(ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

int fmha_mxfp8_selftest_bounded_wait(uint32_t budget_us, void* stream, uint32_t* word, float* ms) {
    if (!word || !ms || budget_us == 0 || budget_us > 100000u) return FMHA_MXFP8_E_ARG;   // at most 0.1 s: this is a self-test, not a stall
    int dev = 0, khz = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
    if (e != cudaSuccess) return -static_cast<int>(e);
    const long long cycles = static_cast<long long>(budget_us) * (khz > 0 ? khz : 1965000) / 1000;
    e = b200mx::run_bounded_wait_selftest(cycles, static_cast<cudaStream_t>(stream), word, ms);
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

}  // extern "C"
