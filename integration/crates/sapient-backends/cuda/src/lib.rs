//! `CudaForwardEngine`: the resident B200 decoder behind the interface sapient's other GPU engine exposes
//! (`WgpuForwardEngine`, crates/sapient-models/src/forward/wgpu_engine.rs:93-110,173-341,343-360,635-676), so
//! `ForwardEngine` can carry it as one more variant and every caller — `Pipeline`, `SpeculativePipeline`, the server —
//! keeps working unchanged.
//!
//! All device work happens inside libsapient_cuda.so; this file only marshals arguments and maps status codes to
//! `anyhow` errors. No unwinding crosses the boundary (the workspace builds with `panic = "abort"`).
//!
//! NOT COMPILED where this file was written (no Rust toolchain there); it is written against the reference's
//! interfaces as read from its sources.
mod ffi;

use std::collections::HashMap;
use std::ffi::{CStr, CString};
use std::path::Path;

use anyhow::{bail, Context, Result};
use sapient_core::{DType, Tensor};
use sapient_hub::model_info::{ArchType, ModelInfo};

pub use ffi::SpModelDesc;

/// How the engine is placed: one GPU, or one rank of a tensor-parallel group (one process per GPU).
#[derive(Debug, Clone, Copy)]
pub struct CudaPlacement {
    pub device: i32,
    pub tp_rank: i32,
    pub tp_size: i32,
    /// Sequence slots (1 = the reference's single-sequence engine).
    pub max_batch: i32,
}

impl Default for CudaPlacement {
    fn default() -> Self {
        Self { device: 0, tp_rank: 0, tp_size: 1, max_batch: 1 }
    }
}

pub struct CudaForwardEngine {
    raw: *mut ffi::SpEngine,
    vocab: usize,
    /// Rows of the logit buffers this rank receives (the whole vocabulary on one GPU).
    vocab_local: usize,
}

// One engine is never entered by two threads at once (callers hold it behind `Arc<Mutex<..>>` as they do for the
// other engines); the library sets the device on every entry, so the calling OS thread may change between calls.
unsafe impl Send for CudaForwardEngine {}

fn check(status: i32) -> Result<()> {
    if status == ffi::SP_OK {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(ffi::sp_cuda_last_error()) }.to_string_lossy().into_owned();
    let kind = match status {
        ffi::SP_ERR_SHAPE => "shape mismatch",
        ffi::SP_ERR_DTYPE => "unsupported dtype",
        ffi::SP_ERR_OOM => "out of device memory",
        ffi::SP_ERR_CUDA => "CUDA error",
        ffi::SP_ERR_KV_FULL => "KV cache full",
        ffi::SP_ERR_COMM => "tensor-parallel peer did not arrive",
        ffi::SP_ERR_ARG => "bad argument",
        ffi::SP_ERR_VOCAB => "token id out of range",
        ffi::SP_ERR_STATE => "engine not ready",
        ffi::SP_ERR_IO => "GGUF unreadable",
        _ => "error",
    };
    bail!("cuda backend: {kind}: {msg}")
}

/// ggml type code + the bytes to hand over for one tensor of the HF-named weight map.
fn tensor_payload(t: &Tensor) -> Result<(i32, &[u8])> {
    Ok(match t.dtype() {
        DType::F32 => (ffi::SP_F32, t.as_bytes()),
        DType::F16 => (ffi::SP_F16, t.as_bytes()),
        DType::BF16 => (ffi::SP_BF16, t.as_bytes()),
        DType::Q4_0 => (ffi::SP_Q4_0, t.as_quant_blocks()),
        DType::Q8_0 => (ffi::SP_Q8_0, t.as_quant_blocks()),
        DType::Q4_K => (ffi::SP_Q4_K, t.as_quant_blocks()),
        DType::Q5_K => (ffi::SP_Q5_K, t.as_quant_blocks()),
        DType::Q6_K => (ffi::SP_Q6_K, t.as_quant_blocks()),
        other => bail!("cuda backend: tensor dtype {other} is not supported"),
    })
}

fn desc_from_info(info: &ModelInfo, place: CudaPlacement, max_ctx: usize) -> Result<SpModelDesc> {
    let arch = match info.arch {
        ArchType::Llama | ArchType::Qwen => 0,
        // Phi-3 / 3.5 / 4-mini run PhiForward's sequential RMSNorm + SwiGLU block (forward/phi.rs:391-503), which is the
        // engine's Llama block; the fused `mlp.gate_up_proj` tensor is cut at upload
        ArchType::Phi if info.model_type == "phi3" => 0,
        ArchType::Phi => 1,
        other => bail!("CudaForwardEngine supports Llama / Qwen2 / Phi-2 decoders (got {other:?})"),
    };
    if info.is_moe() {
        bail!("CudaForwardEngine does not run mixture-of-experts models");
    }
    let rotary_dim = ((info.head_dim as f64) * info.partial_rotary_factor).round() as i32;
    Ok(SpModelDesc {
        arch,
        n_layers: info.num_hidden_layers as i32,
        hidden: info.hidden_size as i32,
        n_heads: info.num_attention_heads as i32,
        n_kv_heads: info.num_key_value_heads as i32,
        head_dim: info.head_dim as i32,
        ffn: info.intermediate_size as i32,
        vocab: info.vocab_size as i32,
        max_ctx: max_ctx as i32,
        rotary_dim,
        norm_eps: info.rms_norm_eps as f32,
        rope_theta: info.rope_theta as f32,
        max_batch: place.max_batch,
        max_tokens: 512,
        device: place.device,
        tp_rank: place.tp_rank,
        tp_size: place.tp_size,
        kv_pages: 0,
    })
}

impl CudaForwardEngine {
    /// `from_weights(info, weights)`: consumes the HF-named map the GGUF loader produces, like
    /// `WgpuForwardEngine::from_weights` (wgpu_engine.rs:173-186). Quantised tensors keep their block format on the
    /// device; F16 / BF16 matrices are re-quantised to Q8_0 at upload as the CPU engines do (forward/common.rs:39-86).
    pub fn from_weights(info: ModelInfo, weights: HashMap<String, Tensor>) -> Result<Self> {
        let max_ctx = kv_cache_ctx(info.max_position_embeddings);
        Self::from_weights_placed(info, weights, CudaPlacement::default(), max_ctx)
    }

    pub fn from_weights_placed(
        info: ModelInfo,
        weights: HashMap<String, Tensor>,
        place: CudaPlacement,
        max_ctx: usize,
    ) -> Result<Self> {
        if unsafe { ffi::sp_cuda_device_count() } <= place.device {
            bail!("cuda backend: device {} not present", place.device);
        }
        check(unsafe { ffi::sp_cuda_check_kernels(place.device) }).context("this build targets sm_100a (B200)")?;
        let desc = desc_from_info(&info, place, max_ctx)?;
        let mut raw = std::ptr::null_mut();
        check(unsafe { ffi::sp_cuda_engine_create(&desc, &mut raw) })?;
        let mut eng = Self { raw, vocab: info.vocab_size, vocab_local: info.vocab_size };
        for (name, t) in &weights {
            let (code, bytes) = tensor_payload(t)?;
            let dims: Vec<i64> = t.shape().dims().iter().map(|&d| d as i64).collect();
            let cname = CString::new(name.as_str())?;
            check(unsafe {
                ffi::sp_cuda_engine_set_tensor(raw, cname.as_ptr(), code, dims.as_ptr(), dims.len() as i32, bytes.as_ptr().cast(), bytes.len())
            })
            .with_context(|| format!("uploading {name}"))?;
        }
        drop(weights); // the device holds the only copy from here on
        check(unsafe { ffi::sp_cuda_engine_finalize(raw) })?;
        eng.read_vocab_local()?;
        Ok(eng)
    }

    /// Reads the GGUF inside the library: mapped file, pinned double-buffered uploads, name map, q/k un-permute and
    /// Phi qkv split as in crates/sapient-models/src/gguf_weights.rs:61-154,273-455.
    pub fn from_gguf(path: &Path, device: i32, max_ctx: usize, max_batch: i32) -> Result<Self> {
        let cpath = CString::new(path.to_string_lossy().as_bytes())?;
        let mut raw = std::ptr::null_mut();
        check(unsafe { ffi::sp_cuda_engine_from_gguf(cpath.as_ptr(), device, max_ctx as i32, max_batch, &mut raw) })?;
        let mut desc = SpModelDesc::default();
        let mut eng = Self { raw, vocab: 0, vocab_local: 0 };
        check(unsafe { ffi::sp_cuda_engine_desc(raw, &mut desc) })?;
        eng.vocab = desc.vocab as usize;
        eng.read_vocab_local()?;
        Ok(eng)
    }

    fn read_vocab_local(&mut self) -> Result<()> {
        let (mut rows, mut first) = (0i32, 0i32);
        check(unsafe { ffi::sp_cuda_engine_vocab_local(self.raw, &mut rows, &mut first) })?;
        self.vocab_local = rows as usize;
        Ok(())
    }

    // ── tensor parallelism: exchange `tp_handle()` of every rank by any transport, then `tp_connect` ──
    pub fn tp_handle(&mut self) -> Result<[u8; ffi::SP_TP_HANDLE_BYTES]> {
        let mut h = [0u8; ffi::SP_TP_HANDLE_BYTES];
        check(unsafe { ffi::sp_cuda_engine_tp_handle(self.raw, h.as_mut_ptr().cast(), h.len()) })?;
        Ok(h)
    }
    pub fn tp_connect(&mut self, handles_in_rank_order: &[u8], n_ranks: i32) -> Result<()> {
        check(unsafe { ffi::sp_cuda_engine_tp_connect(self.raw, handles_in_rank_order.as_ptr().cast(), n_ranks) })
    }
    /// After an `SP_ERR_COMM`: every rank calls this after a host-side barrier to re-align the exchange counters.
    pub fn tp_reset(&mut self) -> Result<()> {
        check(unsafe { ffi::sp_cuda_engine_tp_reset(self.raw) })
    }

    // ── the ForwardEngine surface (forward/mod.rs:381-506) ──
    pub fn reset_cache(&mut self) {
        unsafe { ffi::sp_cuda_reset_cache(self.raw, -1) };
    }

    pub fn truncate_cache(&mut self, n: usize) -> usize {
        let mut kept = 0usize;
        unsafe { ffi::sp_cuda_truncate_cache(self.raw, 0, n, &mut kept) };
        kept
    }

    pub fn forward_logits(&mut self, input_ids: &[u32], use_cache: bool) -> Result<Vec<f32>> {
        let mut out = vec![0f32; self.vocab_local];
        check(unsafe { ffi::sp_cuda_forward_logits(self.raw, input_ids.as_ptr(), input_ids.len(), use_cache as i32, out.as_mut_ptr()) })?;
        Ok(out)
    }

    pub fn forward_all_logits(&mut self, input_ids: &[u32]) -> Result<Vec<Vec<f32>>> {
        let mut flat = vec![0f32; input_ids.len() * self.vocab_local];
        check(unsafe { ffi::sp_cuda_forward_all_logits(self.raw, input_ids.as_ptr(), input_ids.len(), flat.as_mut_ptr()) })?;
        Ok(flat.chunks(self.vocab_local).map(<[f32]>::to_vec).collect())
    }

    pub fn forward_all_logits_cached(&mut self, input_ids: &[u32]) -> Result<Vec<Vec<f32>>> {
        let mut flat = vec![0f32; input_ids.len() * self.vocab_local];
        check(unsafe { ffi::sp_cuda_forward_all_logits_cached(self.raw, input_ids.as_ptr(), input_ids.len(), flat.as_mut_ptr()) })?;
        Ok(flat.chunks(self.vocab_local).map(<[f32]>::to_vec).collect())
    }

    /// Greedy decoding with the loop on the device: `steps` tokens after `first`, no logits cross the bus. This is what
    /// `Pipeline::generate_*` does with `SamplingStrategy::Greedy` (crates/sapient-generate/src/pipeline.rs:540-659).
    pub fn decode_greedy(&mut self, first: u32, steps: usize) -> Result<Vec<u32>> {
        let mut out = vec![0u32; steps];
        let slot = 0i32;
        check(unsafe { ffi::sp_cuda_decode_greedy(self.raw, &first, &slot, 1, steps as i32, out.as_mut_ptr()) })?;
        Ok(out)
    }

    pub fn embed(&mut self, _input_ids: &[u32]) -> Result<Vec<f32>> {
        bail!("embed() is not supported on the cuda backend")
    }

    pub fn is_hybrid(&self) -> bool {
        false
    }

    pub fn backend_label(&self) -> String {
        let mut buf = [0 as std::os::raw::c_char; 96];
        if unsafe { ffi::sp_cuda_backend_label(self.raw, buf.as_mut_ptr(), buf.len()) } != ffi::SP_OK {
            return "cuda".into();
        }
        unsafe { CStr::from_ptr(buf.as_ptr()) }.to_string_lossy().into_owned()
    }

    pub(crate) fn raw(&mut self) -> *mut ffi::SpEngine {
        self.raw
    }
}

impl Drop for CudaForwardEngine {
    fn drop(&mut self) {
        unsafe { ffi::sp_cuda_engine_destroy(self.raw) }
    }
}

/// Greedy speculative decoding with both loops inside the library: the schedule of `SpeculativePipeline` at
/// temperature 0 (crates/sapient-generate/src/speculative.rs:499-631) with one k+1-row verify per round.
/// Returns the generated tokens and (rounds, drafted, accepted).
pub fn spec_greedy(
    target: &mut CudaForwardEngine,
    draft: &mut CudaForwardEngine,
    prompt: &[u32],
    k: usize,
    max_new: usize,
    eos: &[u32],
) -> Result<(Vec<u32>, [u64; 3])> {
    let mut out = vec![0u32; max_new];
    let mut n_out = 0usize;
    let mut stats = [0u64; 3];
    check(unsafe {
        ffi::sp_cuda_spec_greedy(
            target.raw(),
            draft.raw(),
            prompt.as_ptr(),
            prompt.len(),
            k as i32,
            max_new,
            eos.as_ptr(),
            eos.len() as i32,
            out.as_mut_ptr(),
            &mut n_out,
            stats.as_mut_ptr(),
        )
    })?;
    out.truncate(n_out);
    Ok((out, stats))
}

/// Continuous batching over one engine's sequence slots (greedy generations; prompt prefixes shared on reference-counted
/// KV pages). The reference serves one sequence per engine (crates/sapient-generate/src/pipeline.rs:540-659) and lists
/// batching as future work (docs/ROADMAP.md:312); a server's request loop calls `step` while anything is queued or running.
pub struct CudaBatcher {
    raw: *mut ffi::SpBatcher,
    /// The batcher drives this engine; it stays alive (and must not be used directly) as long as the batcher does.
    _engine: Box<CudaForwardEngine>,
}

unsafe impl Send for CudaBatcher {}

impl CudaBatcher {
    pub fn new(mut engine: Box<CudaForwardEngine>, prefill_chunk: usize, prefix_cache: bool) -> Result<Self> {
        let mut raw = std::ptr::null_mut();
        check(unsafe { ffi::sp_cuda_batcher_create(engine.raw(), prefill_chunk as i32, prefix_cache as i32, &mut raw) })?;
        Ok(Self { raw, _engine: engine })
    }

    /// Queues a generation; the id names it in `poll` / `cancel` / `forget`.
    pub fn submit(&mut self, prompt: &[u32], max_new: usize, eos: &[u32]) -> Result<u64> {
        let mut id = 0u64;
        check(unsafe {
            ffi::sp_cuda_batcher_submit(self.raw, prompt.as_ptr(), prompt.len(), max_new, eos.as_ptr(), eos.len() as i32, &mut id)
        })?;
        Ok(id)
    }

    /// One scheduler iteration (admit, a bounded prefill chunk, one decode step); returns (running, waiting).
    pub fn step(&mut self) -> Result<(usize, usize)> {
        let (mut r, mut w) = (0i32, 0i32);
        check(unsafe { ffi::sp_cuda_batcher_step(self.raw, &mut r, &mut w) })?;
        Ok((r as usize, w as usize))
    }

    /// Tokens generated so far and whether the request has left the batch.
    pub fn poll(&self, id: u64) -> Result<(Vec<u32>, bool)> {
        let (mut n, mut fin) = (0usize, 0i32);
        check(unsafe { ffi::sp_cuda_batcher_poll(self.raw, id, std::ptr::null_mut(), 0, &mut n, &mut fin) })?;
        let mut out = vec![0u32; n];
        check(unsafe { ffi::sp_cuda_batcher_poll(self.raw, id, out.as_mut_ptr(), out.len(), &mut n, &mut fin) })?;
        out.truncate(n);
        Ok((out, fin != 0))
    }

    pub fn cancel(&mut self, id: u64) -> Result<()> {
        check(unsafe { ffi::sp_cuda_batcher_cancel(self.raw, id) })
    }

    pub fn forget(&mut self, id: u64) -> Result<()> {
        check(unsafe { ffi::sp_cuda_batcher_forget(self.raw, id) })
    }
}

impl Drop for CudaBatcher {
    fn drop(&mut self) {
        unsafe { ffi::sp_cuda_batcher_destroy(self.raw) } // before the engine it drives
    }
}

/// The context window the CPU engines allocate (kv_cache_ctx, crates/sapient-models/src/forward/common.rs:25-37):
/// min(model maximum, SAPIENT_CTX or 8192). Restated here because that function is private to sapient-models; when this
/// crate is wired in, call the original instead.
fn kv_cache_ctx(model_max: usize) -> usize {
    let cap = std::env::var("SAPIENT_CTX").ok().and_then(|v| v.parse::<usize>().ok()).filter(|&v| v > 0).unwrap_or(8192);
    model_max.min(cap).max(1)
}
