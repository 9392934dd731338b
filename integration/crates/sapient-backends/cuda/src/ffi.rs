//! Raw declarations of include/sapient_cuda.h — the entries the engine path, the speculative loop and the
//! tensor-parallel set-up use. Argument order and types follow the header one to one.
#![allow(non_camel_case_types, dead_code)]
use std::os::raw::{c_char, c_void};

#[repr(C)]
pub struct SpEngine {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct SpWeight {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct SpBatcher {
    _opaque: [u8; 0],
}

pub const SP_OK: i32 = 0;
pub const SP_ERR_SHAPE: i32 = 1;
pub const SP_ERR_DTYPE: i32 = 2;
pub const SP_ERR_OOM: i32 = 3;
pub const SP_ERR_CUDA: i32 = 4;
pub const SP_ERR_KV_FULL: i32 = 5;
pub const SP_ERR_COMM: i32 = 6;
pub const SP_ERR_ARG: i32 = 7;
pub const SP_ERR_VOCAB: i32 = 8;
pub const SP_ERR_STATE: i32 = 9;
pub const SP_ERR_IO: i32 = 10;

/// ggml tensor type codes (crates/sapient-io/src/gguf.rs:88-129)
pub const SP_F32: i32 = 0;
pub const SP_F16: i32 = 1;
pub const SP_Q4_0: i32 = 2;
pub const SP_Q8_0: i32 = 8;
pub const SP_Q4_K: i32 = 12;
pub const SP_Q5_K: i32 = 13;
pub const SP_Q6_K: i32 = 14;
pub const SP_BF16: i32 = 30;

pub const SP_TP_HANDLE_BYTES: usize = 64;

/// 80 bytes; the field order is the header's.
#[repr(C)]
#[derive(Debug, Default, Clone, Copy)]
pub struct SpModelDesc {
    pub arch: i32,
    pub n_layers: i32,
    pub hidden: i32,
    pub n_heads: i32,
    pub n_kv_heads: i32,
    pub head_dim: i32,
    pub ffn: i32,
    pub vocab: i32,
    pub max_ctx: i32,
    pub rotary_dim: i32,
    pub norm_eps: f32,
    pub rope_theta: f32,
    pub max_batch: i32,
    pub max_tokens: i32,
    pub device: i32,
    pub tp_rank: i32,
    pub tp_size: i32,
    pub kv_pages: i64,
}

extern "C" {
    pub fn sp_cuda_last_error() -> *const c_char;
    pub fn sp_cuda_device_count() -> i32;
    pub fn sp_cuda_check_kernels(device: i32) -> i32;

    pub fn sp_cuda_engine_create(desc: *const SpModelDesc, out: *mut *mut SpEngine) -> i32;
    pub fn sp_cuda_engine_set_tensor(
        e: *mut SpEngine,
        hf_name: *const c_char,
        dtype: i32,
        dims: *const i64,
        ndim: i32,
        bytes: *const c_void,
        nbytes: usize,
    ) -> i32;
    pub fn sp_cuda_engine_finalize(e: *mut SpEngine) -> i32;
    pub fn sp_cuda_engine_from_gguf(
        path: *const c_char,
        device: i32,
        max_ctx: i32,
        max_batch: i32,
        out: *mut *mut SpEngine,
    ) -> i32;
    pub fn sp_cuda_engine_desc(e: *const SpEngine, out: *mut SpModelDesc) -> i32;
    pub fn sp_cuda_engine_destroy(e: *mut SpEngine);
    pub fn sp_cuda_engine_load_stats(e: *const SpEngine, seconds: *mut f64, bytes: *mut u64) -> i32;
    pub fn sp_cuda_engine_resident_bytes(e: *const SpEngine, weights: *mut u64, kv: *mut u64) -> i32;

    pub fn sp_cuda_engine_tp_handle(e: *mut SpEngine, out: *mut c_void, cap: usize) -> i32;
    pub fn sp_cuda_engine_tp_connect(e: *mut SpEngine, handles: *const c_void, n_ranks: i32) -> i32;
    pub fn sp_cuda_engine_vocab_local(e: *const SpEngine, rows: *mut i32, first: *mut i32) -> i32;
    pub fn sp_cuda_engine_tp_set_wait_ms(e: *mut SpEngine, ms: i32) -> i32;
    pub fn sp_cuda_engine_tp_reset(e: *mut SpEngine) -> i32;

    pub fn sp_cuda_engine_set_kv_rounding(e: *mut SpEngine, mode: i32) -> i32;
    pub fn sp_cuda_engine_set_large_m_gemm(e: *mut SpEngine, on: i32) -> i32;
    pub fn sp_cuda_engine_set_graphs(e: *mut SpEngine, on: i32) -> i32;
    pub fn sp_cuda_engine_synchronize(e: *mut SpEngine) -> i32;

    pub fn sp_cuda_forward_logits(e: *mut SpEngine, ids: *const u32, n: usize, use_cache: i32, logits_out: *mut f32) -> i32;
    pub fn sp_cuda_forward_all_logits(e: *mut SpEngine, ids: *const u32, n: usize, out: *mut f32) -> i32;
    pub fn sp_cuda_forward_all_logits_cached(e: *mut SpEngine, ids: *const u32, n: usize, out: *mut f32) -> i32;
    pub fn sp_cuda_forward_slot(
        e: *mut SpEngine,
        slot: i32,
        ids: *const u32,
        n: usize,
        all_positions: i32,
        logits_out: *mut f32,
    ) -> i32;
    pub fn sp_cuda_decode_batch(
        e: *mut SpEngine,
        ids: *const u32,
        slots: *const i32,
        b: i32,
        logits_out: *mut f32,
        argmax_out: *mut u32,
    ) -> i32;
    pub fn sp_cuda_decode_greedy(
        e: *mut SpEngine,
        first_ids: *const u32,
        slots: *const i32,
        b: i32,
        steps: i32,
        tokens_out: *mut u32,
    ) -> i32;
    pub fn sp_cuda_spec_greedy(
        target: *mut SpEngine,
        draft: *mut SpEngine,
        prompt: *const u32,
        n_prompt: usize,
        k: i32,
        max_new: usize,
        eos_ids: *const u32,
        n_eos: i32,
        tokens_out: *mut u32,
        n_out: *mut usize,
        stats: *mut u64,
    ) -> i32;

    pub fn sp_cuda_engine_slot_page(e: *const SpEngine, slot: i32, index: i32, page: *mut i32) -> i32;
    pub fn sp_cuda_engine_adopt_prefix(e: *mut SpEngine, slot: i32, pages: *const i32, n: i32) -> i32;

    pub fn sp_cuda_batcher_create(e: *mut SpEngine, prefill_chunk: i32, prefix_cache: i32, out: *mut *mut SpBatcher) -> i32;
    pub fn sp_cuda_batcher_destroy(b: *mut SpBatcher);
    pub fn sp_cuda_batcher_submit(
        b: *mut SpBatcher,
        prompt: *const u32,
        n: usize,
        max_new: usize,
        eos_ids: *const u32,
        n_eos: i32,
        id: *mut u64,
    ) -> i32;
    pub fn sp_cuda_batcher_step(b: *mut SpBatcher, n_running: *mut i32, n_waiting: *mut i32) -> i32;
    pub fn sp_cuda_batcher_poll(
        b: *const SpBatcher,
        id: u64,
        tokens_out: *mut u32,
        cap: usize,
        n_tokens: *mut usize,
        finished: *mut i32,
    ) -> i32;
    pub fn sp_cuda_batcher_cancel(b: *mut SpBatcher, id: u64) -> i32;
    pub fn sp_cuda_batcher_forget(b: *mut SpBatcher, id: u64) -> i32;
    pub fn sp_cuda_batcher_stats(b: *const SpBatcher, out: *mut u64, cap: i32) -> i32;

    pub fn sp_cuda_reset_cache(e: *mut SpEngine, slot: i32) -> i32;
    pub fn sp_cuda_truncate_cache(e: *mut SpEngine, slot: i32, n: usize, kept: *mut usize) -> i32;
    pub fn sp_cuda_seq_len(e: *const SpEngine, slot: i32, len: *mut usize) -> i32;
    pub fn sp_cuda_backend_label(e: *const SpEngine, buf: *mut c_char, cap: usize) -> i32;
}
