/*
 * C ABI of the B200 (sm_100a) implementation of the MXFP8 attention forward path, head dim 128:
 * the four kernels fmha_fwd_hd128_mxfp8_v3_{vs128, t128, kvsplit, kvsplit_combine8h} and the
 * shape-based dispatch that selects between them.
 *
 * The structs below are byte-for-byte the packed kernel-argument blocks that the reference's
 * `amdc gen-host` emits (tests/gpu/generated/fmha_fwd_hd128_mxfp8_v3_*_abi.h), so a caller that
 * fills the reference's `Args` can pass the same bytes here. Everything is plain C: pointers,
 * integers, no C++ or framework types. All device pointers are CUDA device pointers owned by the
 * caller; nothing in this library allocates device memory on the launch path.
 *
 * Return codes of every function that returns int: 0 = ok; > 0 = a host-contract class
 * (FMHA_MXFP8_E_*); < 0 = minus a cudaError_t / CUresult value.
 */
#ifndef FMHA_MXFP8_ABI_H
#define FMHA_MXFP8_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Kernel ids, in the order of the reference's shipped list (crates/amdgpu-graph/src/dispatch.rs:513-519). */
enum fmha_mxfp8_kernel {
    FMHA_MXFP8_VS128 = 0,     /* fmha_fwd_hd128_mxfp8_v3_vs128: 256 query rows per logical block */
    FMHA_MXFP8_T128 = 1,      /* fmha_fwd_hd128_mxfp8_v3_t128: 128 query rows per logical block */
    FMHA_MXFP8_KVSPLIT = 2,   /* fmha_fwd_hd128_mxfp8_v3_kvsplit: key range split over grid z, writes partials */
    FMHA_MXFP8_COMBINE8H = 3  /* fmha_fwd_hd128_mxfp8_v3_kvsplit_combine8h: merges the partials */
};

/* Host-contract failure classes: the reference's GV-HOST-* codes (…_kvsplit_abi.h:186-226). */
enum fmha_mxfp8_error {
    FMHA_MXFP8_OK = 0,
    FMHA_MXFP8_E_EXTENT = 1,   /* GV-HOST-EXTENT   */
    FMHA_MXFP8_E_KA_RANGE = 2, /* GV-HOST-KA-RANGE */
    FMHA_MXFP8_E_KA_IS = 3,    /* GV-HOST-KA-IS    */
    FMHA_MXFP8_E_GRID = 4,     /* GV-HOST-GRID     */
    FMHA_MXFP8_E_SYM = 5,      /* GV-HOST-SYM      */
    FMHA_MXFP8_E_ARG = 6,      /* bad kernel id / null pointer (no reference counterpart) */
    FMHA_MXFP8_E_DEVICE = 7    /* a kernel reported a bounded wait that ran out (see fmha_mxfp8_device_status) */
};

/* Bits of `ext_flags` (offset 0x058, padding in the reference's Args, so 0 = reference behaviour). */
#define FMHA_MXFP8_FLAG_V_BLOCKSCALE 0x1u /* V carries one E8M0 per 32 keys per column at ext_ptr_v_blockscale (extension) */
#define FMHA_MXFP8_FLAG_EXACT_REBASE 0x2u /* move the softmax reference on every tile (the short-sequence recipe) for any length */
#define FMHA_MXFP8_FLAG_TRACE_STAMPS_ONLY 0x4u /* with a trace buffer attached: record the time stamps but not the tile dumps */
/*
 * Causal mask (extension: the reference's MXFP8 kernels have none; the rule is the one of its per-tensor sibling family,
 * crates/amdgpu-stage/src/attention/attn3.rs:298-306): key k is visible to query row i when k < min(i + SK - S + 1, SK), i.e. the last
 * query row sees every key. Needs SK >= S (every row then sees key 0). Unsplit kernels only: a launch of the kvsplit kernel with this
 * flag, or with SK < S, returns FMHA_MXFP8_E_ARG before anything is launched; fmha_mxfp8_auto runs a causal problem unsplit whatever the
 * shape dispatch says.
 */
#define FMHA_MXFP8_FLAG_CAUSAL 0x8u
/*
 * The kvsplit kernel writes its partials as f32 [splits][rows][128] instead of the default f16 (extension; for partials that travel
 * between GPUs before they are combined). The reference's partials are f16 in an allocation sized for f32
 * (crates/amdgpu-kernels/src/fmha/io.rs:83-85); either form fits the contract's `ptr_ohat` extent. Pair it with
 * fmha_mxfp8_combine_f32; fmha_mxfp8_launch(COMBINE8H) reads f16 partials, like the reference's combine8h.
 */
#define FMHA_MXFP8_FLAG_F32_PARTIALS 0x10u
/*
 * Launch detail (extension): when the last round of work items fills at most half of the SMs and an item has at least 48 key tiles, the
 * kernels cut those items in two key ranges and let pairs of CTAs (a cluster of two) merge the halves through distributed shared
 * memory. This flag keeps every item whole. Results agree to f32 summation order either way.
 */
#define FMHA_MXFP8_FLAG_NO_TAIL_SPLIT 0x20u
/*
 * Fused merge (extension; the reference tried the same idea as its "last arriver" combine, tests/gpu/ref_host.cpp:489-497, and kept the
 * two-kernel form): the kvsplit kernel also produces the final bf16 output at `ptr_o`, so no combine8h launch follows. Every CTA that has
 * stored a partial of a 128-row block adds one to the block's counter; the CTA that completes the count merges the block's partials with
 * the arithmetic of combine8h (same bits). Needs `ext_ptr_fused_counters` of the kvsplit Args: uint32 [B * H * ceil(S / 128)], zero
 * before the first launch that uses them; a launch that ends with status 0 leaves them zero. f16 partials only (not with
 * FMHA_MXFP8_FLAG_F32_PARTIALS or a peer plan), at most 8 splits; such a launch is refused with FMHA_MXFP8_E_ARG otherwise. With this bit
 * in fmha_mxfp8_problem.flags, fmha_mxfp8_auto keeps the counters behind the f16 partials in `ws_ohat` (the allocation is sized for f32)
 * and clears them in front of every call; the bit is ignored when the path is not kvsplit.
 */
#define FMHA_MXFP8_FLAG_FUSED_COMBINE 0x40u

#pragma pack(push, 1)
/*
 * Kernel arguments of vs128 and t128: replaces amdc_hostgen::fmha_fwd_hd128_mxfp8_v3_vs128::Args
 * (tests/gpu/generated/fmha_fwd_hd128_mxfp8_v3_vs128_abi.h:10-66; t128 is identical, …_t128_abi.h:10-66). 656 bytes.
 * The three `ext_` fields live in bytes that are padding (`_pad3`, 0x038-0x05F) in the reference struct.
 */
typedef struct fmha_mxfp8_attn_args {
    void* ptr_o;                 /* 0x000 bf16 O [B,S,H,128] */
    uint8_t _pad0[8];
    void* ptr_q;                 /* 0x010 e4m3 Q [B,S,H,128] */
    uint8_t _pad1[8];
    void* ptr_k;                 /* 0x020 e4m3 K [B,SK,HK,128] */
    uint8_t _pad2[8];
    void* ptr_v;                 /* 0x030 e4m3 V [B,SK,HK,128] */
    void* ext_ptr_peer_plan;     /* 0x038 kvsplit only (ignored here): see fmha_mxfp8_peer_plan_build */
    void* ext_ptr_lse;           /* 0x040 optional f32 [B,H,S] natural-log LSE output; NULL = not written */
    void* ext_ptr_v_blockscale;  /* 0x048 optional E8M0 [B,ceil(SK/32),HK,128] V block scales (FMHA_MXFP8_FLAG_V_BLOCKSCALE) */
    uint8_t _pad3b[8];           /* 0x050 the vendor ABI's f32 softmax scale; never read (the scale is folded into Q) */
    uint32_t ext_flags;          /* 0x058 */
    uint8_t _pad3c[4];
    uint32_t s_seq_len;          /* 0x060 S */
    uint8_t _pad4[12];
    uint32_t s_Seqs;             /* 0x070 Q row stride in bytes = H*128 */
    uint8_t _pad5[28];
    uint32_t s_Hs;               /* 0x090 = 128 */
    uint8_t _pad6[12];
    uint32_t s_Bs;               /* 0x0A0 Q batch stride = S*H*128 */
    uint8_t _pad7[12];
    uint32_t s_gqa;              /* 0x0B0 H / HK, power of two in 1..16 */
    uint8_t _pad8[12];
    uint32_t s_k_Seqs;           /* 0x0C0 = HK*128 */
    uint8_t _pad9[12];
    uint32_t s_k_Hs;             /* 0x0D0 = 128 */
    uint8_t _pad10[12];
    uint32_t s_k_Bs;             /* 0x0E0 = SK*HK*128 */
    uint8_t _pad11[44];
    uint32_t s_kv_seq_len;       /* 0x110 SK */
    uint8_t _pad12[44];
    uint32_t s_q_head_num;       /* 0x140 H */
    uint8_t _pad13[12];
    uint32_t s_v_Seqs;           /* 0x150 */
    uint8_t _pad14[12];
    uint32_t s_v_Hs;             /* 0x160 */
    uint8_t _pad15[12];
    uint32_t s_v_Bs;             /* 0x170 */
    uint8_t _pad16[12];
    uint32_t s_o_Seqs;           /* 0x180 = H*256 */
    uint8_t _pad17[12];
    uint32_t s_o_Hs;             /* 0x190 = 256 */
    uint8_t _pad18[12];
    uint32_t s_o_Bs;             /* 0x1A0 = S*H*256 */
    uint8_t _pad19[92];
    void* ptr_q_descale;         /* 0x200 E8M0 [B,S,H,4] (+ 2048*H bytes of slack) */
    uint8_t _pad20[8];
    void* ptr_k_descale;         /* 0x210 E8M0 [B,SK,HK,4] (+ 2560*H bytes of slack) */
    uint8_t _pad21[8];
    void* ptr_v_descale;         /* 0x220 one f32 in a buffer of >= 4096 bytes */
    uint8_t _pad22[8];
    uint32_t s_descale_q_Bs;     /* 0x230 = S*H*4 */
    uint8_t _pad23[12];
    uint32_t s_descale_q_Hs;     /* 0x240 = 4 */
    uint8_t _pad24[12];
    uint32_t s_descale_k_Bs;     /* 0x250 = SK*HK*4 */
    uint8_t _pad25[12];
    uint32_t s_descale_k_Hs;     /* 0x260 = 4 */
    uint8_t _pad26[28];
    uint8_t abi_tail[16];        /* 0x280 */
} fmha_mxfp8_attn_args;

/*
 * Kernel arguments of kvsplit: replaces amdc_hostgen::fmha_fwd_hd128_mxfp8_v3_kvsplit::Args
 * (tests/gpu/generated/fmha_fwd_hd128_mxfp8_v3_kvsplit_abi.h:10-72). 648 bytes; same as above up to 0x26F.
 */
typedef struct fmha_mxfp8_kvsplit_args {
    void* ptr_o;
    uint8_t _pad0[8];
    void* ptr_q;
    uint8_t _pad1[8];
    void* ptr_k;
    uint8_t _pad2[8];
    void* ptr_v;
    void* ext_ptr_peer_plan;     /* 0x038 optional: a device plan from fmha_mxfp8_peer_plan_build; the partial rows then go to other GPUs */
    void* ext_ptr_fused_counters; /* 0x040 with FMHA_MXFP8_FLAG_FUSED_COMBINE: uint32 [B * H * ceil(S / 128)] arrival counters, zero on entry; else unused */
    void* ext_ptr_v_blockscale;
    uint8_t _pad3b[8];
    uint32_t ext_flags;
    uint8_t _pad3c[4];
    uint32_t s_seq_len;
    uint8_t _pad4[12];
    uint32_t s_Seqs;
    uint8_t _pad5[28];
    uint32_t s_Hs;
    uint8_t _pad6[12];
    uint32_t s_Bs;
    uint8_t _pad7[12];
    uint32_t s_gqa;
    uint8_t _pad8[12];
    uint32_t s_k_Seqs;
    uint8_t _pad9[12];
    uint32_t s_k_Hs;
    uint8_t _pad10[12];
    uint32_t s_k_Bs;
    uint8_t _pad11[44];
    uint32_t s_kv_seq_len;
    uint8_t _pad12[44];
    uint32_t s_q_head_num;
    uint8_t _pad13[12];
    uint32_t s_v_Seqs;
    uint8_t _pad14[12];
    uint32_t s_v_Hs;
    uint8_t _pad15[12];
    uint32_t s_v_Bs;
    uint8_t _pad16[12];
    uint32_t s_o_Seqs;
    uint8_t _pad17[12];
    uint32_t s_o_Hs;
    uint8_t _pad18[12];
    uint32_t s_o_Bs;
    uint8_t _pad19[92];
    void* ptr_q_descale;
    uint8_t _pad20[8];
    void* ptr_k_descale;
    uint8_t _pad21[8];
    void* ptr_v_descale;
    uint8_t _pad22[8];
    uint32_t s_descale_q_Bs;
    uint8_t _pad23[12];
    uint32_t s_descale_q_Hs;
    uint8_t _pad24[12];
    uint32_t s_descale_k_Bs;
    uint8_t _pad25[12];
    uint32_t s_descale_k_Hs;
    uint8_t _pad26[12];
    void* ptr_ohat;              /* 0x270 partial O [splits][rows_total][128], normalised per split: f16 (f32 with FMHA_MXFP8_FLAG_F32_PARTIALS); sized for f32 either way */
    void* ptr_lse;               /* 0x278 f32 base-2 log-sum-exp, [splits][rows_total] */
    uint32_t kvs_splits;         /* 0x280 2, 4 or 8 (1 is accepted) */
    uint32_t kvs_rows_total;     /* 0x284 B*S*H */
} fmha_mxfp8_kvsplit_args;

/*
 * Kernel arguments of the combine kernel: replaces amdc_hostgen::fmha_fwd_hd128_mxfp8_v3_kvsplit_combine8h::Args
 * (tests/gpu/generated/fmha_fwd_hd128_mxfp8_v3_kvsplit_combine8h_abi.h:10-19). 36 bytes.
 */
typedef struct fmha_mxfp8_combine_args {
    void* ptr_ohat;      /* 0x00 */
    void* ptr_lse;       /* 0x08 */
    void* ptr_out;       /* 0x10 bf16 [rows_total][128] */
    uint32_t rows_total; /* 0x18 */
    uint32_t d;          /* 0x1C = 128 */
    uint32_t splits;     /* 0x20 */
} fmha_mxfp8_combine_args;
#pragma pack(pop)

/* Contract symbols: replaces the per-kernel `Symbols` structs (…_kvsplit_abi.h:137-141). */
typedef struct fmha_mxfp8_symbols {
    int64_t B;  /* batch (kvsplit only; the unsplit kernels take the batch from grid z) */
    int64_t HK; /* KV heads */
    int64_t KL; /* free symbol of the reference's verifier; only its range (>= 0) is checked */
} fmha_mxfp8_symbols;

/* Allocation sizes in bytes of the caller's buffers: replaces the per-kernel `BufferSizes` structs (…_kvsplit_abi.h:142-152, …_combine8h_abi.h:36-40). */
typedef struct fmha_mxfp8_buffer_sizes {
    uint64_t ptr_q, ptr_k, ptr_v, ptr_o;
    uint64_t ptr_q_descale, ptr_k_descale, ptr_v_descale;
    uint64_t ptr_ohat, ptr_lse; /* kvsplit, combine */
    uint64_t ptr_out;           /* combine */
} fmha_mxfp8_buffer_sizes;

/* Name / kernarg size / reference workgroup size of a kernel id (…_abi.json "kernel", "kernarg_size", "workgroup_size"). */
const char* fmha_mxfp8_kernel_name(int kernel);
size_t fmha_mxfp8_kernarg_size(int kernel);
unsigned fmha_mxfp8_workgroup_size(int kernel);

/*
 * Host-contract check: replaces `validate(const Args&, const BufferSizes&, dim3 grid, const Symbols&, std::string* err)`
 * (…_vs128_abi.h:170-204, …_kvsplit_abi.h:186-226, …_combine8h_abi.h:56-66). Same checks in the same order; on the first
 * failure writes "<GV-HOST-CODE>: <message>" into err (if non-NULL, NUL-terminated, at most cap bytes) and returns the class.
 * `grid` is the reference's logical grid: (ceil(S/256 or 128), H, B or B*splits); the combine kernel's grid is not checked.
 */
int fmha_mxfp8_validate(int kernel, const void* args, const fmha_mxfp8_buffer_sizes* sizes, const uint32_t grid[3],
                        const fmha_mxfp8_symbols* syms, char* err, size_t cap);

/* The logical grid a kernel expects: replaces `grid(const Args&, const Symbols&)` (…_kvsplit_abi.h:234) and, for the combine
 * kernel, ceil(rows_total*128 / (256*8)) (tests/gpu/ref_host.cpp:510-515). */
int fmha_mxfp8_grid(int kernel, const void* args, const fmha_mxfp8_symbols* syms, uint32_t grid[3]);

/*
 * Enqueue one kernel on a CUDA stream: replaces `launch(hipFunction_t, const Args&, dim3 grid, dim3 block, size_t lds, hipStream_t)`
 * (…_vs128_abi.h:205-210). `grid` is the logical grid above; the physical CTA grid is this library's business. `args` is read
 * before the call returns. `stream` is a cudaStream_t (NULL = default stream). Does not validate: call fmha_mxfp8_validate first.
 * One restriction beyond the contract: s_gqa must be a power of two that divides s_q_head_num (the kernels find the KV head with a
 * shift, as crates/amdgpu-stage/src/components.rs:8-17 does); any other group size is refused with FMHA_MXFP8_E_KA_RANGE.
 */
int fmha_mxfp8_launch(int kernel, const void* args, const uint32_t grid[3], void* stream);

/*
 * Shape -> path: replaces `mxfp8_prefill_path(b, h, s, sk) -> (path, splits)` (crates/amdgpu-graph/src/dispatch.rs:494-511,
 * mirrored in tests/gpu/ref_host.cpp:124-155). *path is FMHA_MXFP8_VS128, _T128 or _KVSPLIT; *splits is 0, 2 or 4.
 */
void fmha_mxfp8_dispatch(uint64_t b, uint64_t h, uint64_t s, uint64_t sk, int* path, uint32_t* splits);

/* Tensors and workspaces of one forward call, all device pointers, packed BSHD as the contract demands. */
typedef struct fmha_mxfp8_problem {
    uint32_t B, H, HK, S, SK;
    const void* q;          /* e4m3 [B,S,H,128] */
    const void* k;          /* e4m3 [B,SK,HK,128] */
    const void* v;          /* e4m3 [B,SK,HK,128] */
    const void* q_descale;  /* E8M0 [B,S,H,4]   + slack, q_descale_bytes in total */
    const void* k_descale;  /* E8M0 [B,SK,HK,4] + slack, k_descale_bytes in total */
    const void* v_descale;  /* f32, v_descale_bytes >= 4096 */
    void* out;              /* bf16 [B,S,H,128] */
    uint64_t q_descale_bytes, k_descale_bytes, v_descale_bytes;
    void* ws_ohat;          /* kvsplit workspace, >= splits*B*S*H*512 bytes (may be NULL when the path is not kvsplit) */
    void* ws_lse;           /* kvsplit workspace, >= splits*B*S*H*4 bytes */
    uint64_t ws_ohat_bytes, ws_lse_bytes;
    const void* v_blockscale; /* NULL, or the extension's per-32-key V scales (sets FMHA_MXFP8_FLAG_V_BLOCKSCALE) */
    uint32_t flags;         /* extra FMHA_MXFP8_FLAG_* bits */
} fmha_mxfp8_problem;

/*
 * The whole default path `fmha_fwd_hd128_mxfp8_auto`: dispatch (or a forced path), fill the Args, validate, launch (kvsplit: both
 * kernels, same stream). Mirrors python/amdgpu_jit/ops.py:88-143 (`fmha_fwd_mxfp8`) and tests/gpu/ref_host.cpp:342-397,516-569.
 * path: -1 = auto, else FMHA_MXFP8_VS128 / _T128 / _KVSPLIT; splits: used when path is _KVSPLIT (2, 4 or 8; 0 = 4).
 * On return *path_out / *splits_out (if non-NULL) hold what ran. Allocates nothing.
 */
int fmha_mxfp8_auto(const fmha_mxfp8_problem* prob, int path, uint32_t splits, void* stream, int* path_out, uint32_t* splits_out,
                    char* err, size_t cap);

/*
 * The kvsplit path (split kernel + combine, same stream) with the partials kept in a fixed array inside the library instead of in
 * `ws_ohat` / `ws_lse`, which are ignored. This entry has no counterpart in the reference: there the caller always owns the
 * workspace (tests/gpu/ref_host.cpp:516-569 allocates it per run). It exists for callers that cannot obtain device memory at call
 * time: their memory is already committed to their own pools, or they run where the CUDA allocator must not be entered because it
 * synchronises the device. The call allocates nothing and calls no allocating routine.
 *   - Limit: splits * B * S * H <= FMHA_MXFP8_STATIC_SCRATCH_MAX_ROW_SPLITS (32 MiB of partials + 256 KiB of log-sum-exps per
 *     device); beyond it the call returns FMHA_MXFP8_E_EXTENT with a message and launches nothing.
 *   - The first call on a device resolves the array's address (cudaGetSymbolAddress; may load the module), and the first launch of a
 *     kernel variant on a device sets its shared-memory attribute: make one call per recipe you will use (SK < 512 or not) at start-up,
 *     before any stream capture.
 *   - All calls on a device share the one array: calls that may overlap in time race on it and must be ordered by the caller.
 *   - Nothing in the array needs clearing: every partial the combine reads is written by the split kernel of the same call.
 * splits: 2, 4 or 8 (0 = 4). Inputs, output, scale buffers and `flags` are taken from `prob` as in fmha_mxfp8_auto.
 */
#define FMHA_MXFP8_STATIC_SCRATCH_MAX_ROW_SPLITS 65536u
int fmha_mxfp8_kvsplit_static_scratch(const fmha_mxfp8_problem* prob, uint32_t splits, void* stream, char* err, size_t cap);

/*
 * The combine kernel over f32 partials: ohat f32 [splits][rows_total][128], lse f32 [splits][rows_total] (base 2) -> out bf16
 * [rows_total][128]. Same arithmetic as the combine8h kernel behind fmha_mxfp8_launch (crates/amdgpu-tile/src/epilogue.rs:117-146), which
 * reads f16 partials like the reference; this entry is for partials written with FMHA_MXFP8_FLAG_F32_PARTIALS, e.g. after they have been
 * exchanged between GPUs (`splits` = number of key ranges). No counterpart in the reference, which has one GPU and f16 partials only.
 * ohat and out 16-byte aligned. Returns 0, FMHA_MXFP8_E_ARG, or minus a cudaError_t.
 */
int fmha_mxfp8_combine_f32(const void* ohat, const void* lse, void* out, uint32_t rows_total, uint32_t splits, void* stream);

/*
 * Key-range sharding over the GPUs of one node (one process per GPU) without a collective for the partials. None of this has a
 * counterpart in the reference, which is single-GPU; the algebra is its KV split with "split = GPU"
 * (crates/amdgpu-stage/src/components.rs:58-74, crates/amdgpu-tile/src/epilogue.rs:117-146).
 *   peer_alloc / peer_open / peer_close / peer_free: a device buffer other processes of the node can map (CUDA IPC): alloc returns the
 *       pointer and a 64-byte handle to pass to the peers, which open (and later close) it; the owner frees it after the peers closed.
 *   peer_plan_build: GPU d of `world` combines the query rows [d * S / world, (d + 1) * S / world) (S / world a multiple of 128, one batch
 *       element). ohat_recv[d] / lse_recv[d] are GPU d's receive buffers as mapped into this process (this GPU's own for d == rank):
 *       f16 (f32 with f32_partials != 0) [world][S / world][H][128] and f32 [world][S / world * H]. Writes FMHA_MXFP8_PEER_PLAN_BYTES to
 *       `plan_dev` (device memory, 128-byte aligned), to be passed as ext_ptr_peer_plan of a kvsplit launch with kvs_splits = 1 and with
 *       FMHA_MXFP8_FLAG_F32_PARTIALS set exactly when the plan was built for f32 partials (nothing can check that at launch): that launch
 *       stores row block x of its partial to slot [rank] of the receive buffers of GPU x * 128 / (S / world) (TMA tile stores and plain
 *       stores to peer memory; ptr_ohat / ptr_lse are then not written). The ranks must barrier before combining. f16 is the format of the
 *       reference's partials and half the bytes over NVLink; f32 keeps the partials exact to the kernel's accumulators.
 *   combine_scatter: the combine over `rows` rows of `splits` partials (f16, or f32 with f32_partials != 0), each bf16 row stored to all
 *       `n_outs` output buffers at row `row_offset` (the all-gather of the row slices done by the combine's stores). The ranks must barrier before reading.
 *   peer_barrier: the ranks line up on their streams without a collective library: flag_arrays[r] is rank r's array of `world` uint32
 *       arrival flags (in a peer buffer, zero at first) as mapped into this process; one warp tells every rank that this rank has arrived for
 *       the `arrival`-th time (1, 2, ... per plan; release stores at system scope behind a system-scope fence, so what this GPU's earlier kernels
 *       stored to its peers is performed first) and waits, for at most budget_us, until every rank's arrival shows in the own array. A wait
 *       that runs out sets bit 1 of *status_dev (NULL: the library's device status word) and the kernel ends normally.
 *   copy_async: cudaMemcpyAsync device to device (for hosts that hold raw pointers only).
 * Return 0, FMHA_MXFP8_E_ARG, or minus a cudaError_t.
 */
#define FMHA_MXFP8_PEER_HANDLE_BYTES 64
#define FMHA_MXFP8_PEER_MAX_GPUS 8
#define FMHA_MXFP8_PEER_PLAN_BYTES 1152
int fmha_mxfp8_peer_alloc(size_t bytes, void** dev_ptr, void* handle64);
int fmha_mxfp8_peer_open(const void* handle64, void** dev_ptr);
int fmha_mxfp8_peer_close(void* dev_ptr);
int fmha_mxfp8_peer_free(void* dev_ptr);
int fmha_mxfp8_peer_plan_build(uint32_t world, uint32_t rank, uint32_t H, uint32_t S, int f32_partials, void* const* ohat_recv, void* const* lse_recv,
                               void* plan_dev, void* stream);
int fmha_mxfp8_combine_scatter(const void* ohat, int f32_partials, const void* lse, void* const* outs, uint32_t n_outs, uint64_t row_offset, uint32_t rows,
                               uint32_t splits, void* stream);
int fmha_mxfp8_peer_barrier(void* const* flag_arrays, uint32_t world, uint32_t rank, uint32_t arrival, uint32_t budget_us, void* status_dev, void* stream);
int fmha_mxfp8_copy_async(void* dst, const void* src, size_t bytes, void* stream);

/*
 * The quantisers in front of the path: bf16 activations -> the MXFP8 operands the attention kernels take. The reference has no device
 * code for this step : the rule is the one its harness applies on the host (tests/gpu/ref_host.cpp:239-254).
 *   quantize_qk: x bf16 [rows][128] -> out e4m3 [rows][128], scales E8M0 [rows][4] (one per 32 head-dim elements):
 *                E8M0 = clamp(floor(log2 amax(x * mul)) - 8 + 127, 0, 254), element = e4m3_rne_sat(x * mul * 2^-(E8M0 - 127)).
 *                mul = log2(e) / sqrt(128) for Q (the softmax scale the kernels expect folded into Q), 1 for K.
 *                The caller appends the contract's zeroed slack behind `out_scales` itself.
 *   quantize_v:  x bf16 [n_elems] (a multiple of 8) -> out e4m3, v_descale[0] = amax / 448 (1 if the tensor is all zero),
 *                element = e4m3_rne_sat(x / v_descale[0]). v_descale needs 8 writable bytes (the contract's buffer has 4096).
 * f32 arithmetic, one rounding per operation; inputs must be finite. x 16-byte aligned, out 8-byte aligned. Return 0, FMHA_MXFP8_E_ARG,
 * or minus a cudaError_t.
 */
int fmha_mxfp8_quantize_qk(const void* x_bf16, uint64_t rows, float mul, void* out_e4m3, void* out_scales, void* stream);
int fmha_mxfp8_quantize_v(const void* x_bf16, uint64_t n_elems, void* out_e4m3, void* v_descale, void* stream);

/*
 * Device status word: 0 when no kernel of this library ever gave up a bounded wait on the current device, else a bit mask of the
 * roles that did. Synchronises the device. No counterpart in the reference (its kernels have no bounded waits); it stands where
 * the reference harness checks hipDeviceSynchronize() after a launch (tests/gpu/ref_host.cpp:400).
 */
int fmha_mxfp8_device_status(uint32_t* status);

/*
 * Diagnostics hook in the spirit of the reference's stamp buffer (docs/stamps.md): when a device buffer of at least
 * FMHA_MXFP8_TRACE_BYTES is attached, logical block (0,0,0) of the next attention launches records its first score tile, the
 * unnormalised O, the row sums, the row references and per-tile SM-clock stamps of its warp roles there. Pass NULL to detach.
 */
#define FMHA_MXFP8_TRACE_BYTES (4u * (16384u + 16384u + 256u + 4096u + 2048u))
int fmha_mxfp8_trace_attach(void* dev_buf, size_t bytes);

/*
 * Issue-only ceiling of the tensor pipe, the second denominator of the attention kernel's roofline fraction: each of `ctas` CTAs has one
 * thread issue `iters` x 4 tcgen05.mma kind::f8f6f4 (M128 N128 K32, e4m3) back to back on resident operands, four dependent MMAs per
 * tile, tiles alternating between two accumulators (the shape of the Q K^T stream). Writes the elapsed milliseconds (CUDA events on
 * `stream`) and returns 0. No counterpart in the reference (its roofline is the vendor kernel measured in the same run,
 * tools/port_gate.sh:163-187).
 */
int fmha_mxfp8_mma_issue_ceiling(int iters, int ctas, void* stream, float* ms);

/*
 * Self-test of the bounded waits: a one-CTA kernel waits `budget_us` microseconds (1 .. 100000) for an mbarrier arrival that never
 * comes, gives up, and ends normally. *word: bit 0 = the wait ran out, bit 1 = a second warp left its own wait because of the raised
 * flag (both expected: 3), bit 2 = a wait claimed success (never expected). *ms = the kernel's duration (CUDA events). The library's
 * device status word is not touched. Synchronises `stream`. No counterpart in the reference, whose kernels wait without a limit.
 */
int fmha_mxfp8_selftest_bounded_wait(uint32_t budget_us, void* stream, uint32_t* word, float* ms);

#ifdef __cplusplus
}
#endif
#endif /* FMHA_MXFP8_ABI_H */
