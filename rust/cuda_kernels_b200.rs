//! Additive FFI for `libnve_kernels.so` built from this repository: the declarations a maintainer adds beside the
//! existing `extern "C"` block of `src/cuda_kernels.rs` (:57-289), plus wrappers in that file's own style
//! (:296-339 pointer helpers, :525-573 wrapper shape).
//!
//! NOT COMPILED in the environment this repository was written in (no cargo / rustc there).  The C side of every
//! declaration below is exercised through Python ctypes by the test suite; signatures follow `include/nve_kernels.h`
//! Part 2.  Intended use: `include!` it inside `mod inner` of `src/cuda_kernels.rs` (it relies on that module's
//! `stream()`, `cuda_dev_ptr*` helpers and imports), or paste the pieces needed.

/// One matrix of a fused multi-matrix GEMV (`nve_b200_w4_matrix`).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct NveB200W4Matrix {
    pub nibbles: *const u8,                 // [N, K/2]
    pub scales: *const f32,                 // [N, K/32]
    pub out: *mut std::ffi::c_void,         // [N] of out_dtype
    pub residual: *const std::ffi::c_void,  // NULL, or [N] of out_dtype: out = residual + y (may alias out)
    pub n: i32,
}

/// Per-layer descriptor of the persistent decode step (`nve_b200_decode_layer`); lives in DEVICE memory.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct NveB200DecodeLayer {
    pub nibbles: [*const u8; 7], // q, k, v, o, gate, up, down
    pub scales: [*const f32; 7],
    pub awq: [*const f32; 4],    // q/k/v, o, gate/up, down activation multipliers (NULL: none)
    pub input_norm: *const u16,
    pub post_attn_norm: *const u16,
    pub k_cache: *mut u16,
    pub v_cache: *mut u16,
    pub use_w4a8: i32,
    pub reserved: i32,
}

/// Model description of the persistent decode step (`nve_b200_decode_model`); passed by host pointer.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct NveB200DecodeModel {
    pub hidden: i32,
    pub ffn: i32,
    pub num_heads: i32,
    pub num_kv_heads: i32,
    pub head_dim: i32,
    pub max_seq: i32,
    pub num_layers: i32,
    pub norm_eps: f32,
    pub attn_scale: f32,
    pub rope_cos: *const u16,
    pub rope_sin: *const u16,
    pub final_norm: *const u16,
    pub lm_nibbles: *const u8,
    pub lm_scales: *const f32,
    pub logits: *mut f32,
    pub vocab: i32,
    pub lm_use_w4a8: i32,
}

pub const NVE_DT_F16: i32 = 0;
pub const NVE_DT_BF16: i32 = 1;
pub const NVE_DT_F32: i32 = 2;

type Stream = *mut std::ffi::c_void;
type CVoid = std::ffi::c_void;

extern "C" {
    pub fn nve_b200_last_status() -> i32;
    pub fn nve_b200_last_cuda_error() -> i32;
    pub fn nve_b200_launch_count() -> u64;
    pub fn nve_b200_set_pdl(enabled: i32) -> i32;
    /// 0 = tensor-core decode attention where the shape is covered (default), 1 = the CUDA-core kernel whose output
    /// equals the un-fused launch sequence bit for bit; returns the previous setting.
    pub fn nve_b200_set_attn_decode_kernel(mode: i32) -> i32;

    pub fn nve_b200_quantize_q8(x: *const CVoid, xq: *mut i8, scales: *mut f32, k: i32, x_dtype: i32, stream: Stream) -> i32;
    pub fn nve_b200_quantize_q8_awq(x: *const CVoid, awq_inv: *const f32, xq: *mut i8, scales: *mut f32, k: i32,
                                    x_dtype: i32, stream: Stream) -> i32;
    pub fn nve_b200_rmsnorm_quantize_q8(x: *const CVoid, weight: *const CVoid, normed_out: *mut CVoid, xq: *mut i8,
                                        scales: *mut f32, n: i32, eps: f32, dtype: i32, stream: Stream) -> i32;
    pub fn nve_b200_silu_mul_quantize_q8(gate: *const CVoid, up: *const CVoid, mid_out: *mut CVoid, xq: *mut i8,
                                         scales: *mut f32, n: i32, dtype: i32, stream: Stream) -> i32;
    pub fn nve_b200_silu_mul_x16(gate: *const CVoid, up: *const CVoid, mid_out: *mut CVoid, x_lo: *mut u8, x_hi: *mut i8,
                                 x_scales: *mut f32, awq: *const f32, n: i32, dtype: i32, stream: Stream) -> i32;

    pub fn nve_b200_matvec_w4a8_multi(xq: *const i8, xq_scales: *const f32, mats: *const NveB200W4Matrix, num_mats: i32,
                                      k: i32, out_dtype: i32, stream: Stream) -> i32;
    pub fn nve_b200_matvec_w4a16_multi(x: *const CVoid, x_dtype: i32, awq: *const f32, mats: *const NveB200W4Matrix,
                                       num_mats: i32, k: i32, out_dtype: i32, stream: Stream) -> i32;
    pub fn nve_b200_matvec_w4a16_planes_multi(x_lo: *const u8, x_hi: *const i8, x_scales: *const f32,
                                              mats: *const NveB200W4Matrix, num_mats: i32, k: i32, out_dtype: i32,
                                              stream: Stream) -> i32;
    pub fn nve_b200_rmsnorm_matvec_w4a8_multi(h: *const CVoid, norm_weight: *const CVoid, eps: f32, act_dtype: i32,
                                              mats: *const NveB200W4Matrix, num_mats: i32, k: i32, out_dtype: i32,
                                              stream: Stream) -> i32;
    pub fn nve_b200_rmsnorm_matvec_w4a8_awq_multi(h: *const CVoid, norm_weight: *const CVoid, eps: f32, act_dtype: i32,
                                                  awq_inv: *const f32, mats: *const NveB200W4Matrix, num_mats: i32,
                                                  k: i32, out_dtype: i32, stream: Stream) -> i32;
    pub fn nve_b200_rmsnorm_matvec_w4a16_multi(h: *const CVoid, norm_weight: *const CVoid, eps: f32, act_dtype: i32,
                                               awq: *const f32, mats: *const NveB200W4Matrix, num_mats: i32, k: i32,
                                               out_dtype: i32, stream: Stream) -> i32;
    pub fn nve_b200_rmsnorm_gateup_silu_w4a8(h: *const CVoid, norm_weight: *const CVoid, eps: f32, act_dtype: i32,
                                             awq_inv: *const f32, gate: *const NveB200W4Matrix, up: *const NveB200W4Matrix,
                                             mid_out: *mut CVoid, k: i32, stream: Stream) -> i32;
    pub fn nve_b200_rmsnorm_gateup_silu_w4a16(h: *const CVoid, norm_weight: *const CVoid, eps: f32, act_dtype: i32,
                                              awq: *const f32, gate: *const NveB200W4Matrix, up: *const NveB200W4Matrix,
                                              mid_out: *mut CVoid, k: i32, stream: Stream) -> i32;
    pub fn nve_b200_attn_decode_fused_batch(q: *const u16, k_new: *const u16, v_new: *const u16, k_cache: *mut u16,
                                            v_cache: *mut u16, cos_tab: *const u16, sin_tab: *const u16, d_pos: *const i32,
                                            d_seq_len: *const i32, out: *mut u16, batch: i32, num_heads: i32,
                                            num_kv_heads: i32, head_dim: i32, max_seq_len: i32, scale: f32,
                                            stream: Stream) -> i32;
    pub fn nve_b200_rms_norm_rows(x: *const CVoid, weight: *const CVoid, out: *mut CVoid, rows: i32, n: i32, eps: f32,
                                  dtype: i32, stream: Stream) -> i32;
    pub fn nve_b200_add_rms_norm_rows(x: *mut CVoid, delta: *const CVoid, weight: *const CVoid, out: *mut CVoid, rows: i32,
                                      n: i32, eps: f32, dtype: i32, stream: Stream) -> i32;
    pub fn nve_b200_kv_cache_write_rows(k_new: *const u16, k_cache: *mut u16, v_new: *const u16, v_cache: *mut u16,
                                        rows: i32, start_pos: i32, num_kv_heads: i32, head_dim: i32, max_seq_len: i32,
                                        stream: Stream) -> i32;
    pub fn nve_b200_attn_prefill_causal(q: *const u16, k_cache: *const u16, v_cache: *const u16, out: *mut u16, rows: i32,
                                        start_pos: i32, num_heads: i32, num_kv_heads: i32, head_dim: i32,
                                        max_seq_len: i32, scale: f32, stream: Stream) -> i32;
    pub fn nve_b200_rmsnorm_gateup_silu_q8_w4a8(h: *const CVoid, norm_weight: *const CVoid, eps: f32, act_dtype: i32,
                                                awq_inv: *const f32, gate: *const NveB200W4Matrix, up: *const NveB200W4Matrix,
                                                mid_out: *mut CVoid, k: i32, mid_q: *mut i8, mid_scales: *mut f32,
                                                group_counters: *mut u32, stream: Stream) -> i32;
    pub fn nve_b200_rmsnorm_gateup_silu_x16_w4a16(h: *const CVoid, norm_weight: *const CVoid, eps: f32, act_dtype: i32,
                                                  awq: *const f32, gate: *const NveB200W4Matrix, up: *const NveB200W4Matrix,
                                                  mid_out: *mut CVoid, k: i32, mid_lo: *mut u8, mid_hi: *mut i8,
                                                  mid_scales: *mut f32, down_awq: *const f32, group_counters: *mut u32,
                                                  stream: Stream) -> i32;
    pub fn nve_b200_quantize_matvec_w4a8_multi(x: *const CVoid, x_dtype: i32, awq_inv: *const f32,
                                               mats: *const NveB200W4Matrix, num_mats: i32, k: i32, stream: Stream) -> i32;

    pub fn nve_b200_attn_decode_fused(q: *const u16, k_new: *const u16, v_new: *const u16, k_cache: *mut u16,
                                      v_cache: *mut u16, cos_tab: *const u16, sin_tab: *const u16, d_pos: *const i32,
                                      d_seq_len: *const i32, out: *mut u16, out_q: *mut i8, out_scales: *mut f32,
                                      num_heads: i32, num_kv_heads: i32, head_dim: i32, max_seq_len: i32, scale: f32,
                                      stream: Stream) -> i32;

    pub fn nve_b200_gemm_w4a16_scratch_bytes(m: i32, n: i32, k: i32) -> usize;
    pub fn nve_b200_gemm_w4a16(x: *const CVoid, x_dtype: i32, nibbles: *const u8, scales: *const f32, y: *mut CVoid,
                               y_dtype: i32, m: i32, n: i32, k: i32, scratch: *mut CVoid, scratch_bytes: usize,
                               stream: Stream) -> i32;
    pub fn nve_b200_gemm_w4a16_noalloc(x: *const CVoid, x_dtype: i32, nibbles: *const u8, scales: *const f32,
                                       y: *mut CVoid, y_dtype: i32, m: i32, n: i32, k: i32, stream: Stream) -> i32;
    pub fn nve_b200_gemm_error(reset: i32) -> i32;

    pub fn nve_b200_q4_quantize(w: *const f32, awq_scales: *const f32, nibbles: *mut u8, scales: *mut f32, n: i32, k: i32,
                                stream: Stream) -> i32;
    pub fn nve_b200_q4_repack_blocks(cpu_blocks: *const u8, nibbles: *mut u8, scales: *mut f32, n: i32, k: i32,
                                     stream: Stream) -> i32;

    pub fn nve_b200_decode_step_workspace_bytes(model: *const NveB200DecodeModel) -> usize;
    pub fn nve_b200_decode_step_init(workspace: *mut CVoid, workspace_bytes: usize, stream: Stream) -> i32;
    pub fn nve_b200_decode_step(model: *const NveB200DecodeModel, layers_dev: *const NveB200DecodeLayer, hidden: *mut CVoid,
                                d_pos: *const i32, d_seq_len: *const i32, workspace: *mut CVoid, workspace_bytes: usize,
                                stream: Stream) -> i32;
    pub fn nve_b200_decode_step_error(workspace: *mut CVoid, reset: i32) -> i32;

    pub fn nve_b200_tp_create(rank: i32, world: i32, max_rows: i32, handle_out: *mut CVoid) -> i32;
    pub fn nve_b200_tp_connect(handles: *const CVoid) -> i32;
    pub fn nve_b200_tp_error(reset: i32) -> i32;
    pub fn nve_b200_tp_destroy() -> i32;
    pub fn nve_b200_matvec_w4a8_allreduce(xq: *const i8, xq_scales: *const f32, mat: *const NveB200W4Matrix, k: i32,
                                          out_dtype: i32, stream: Stream) -> i32;
    pub fn nve_b200_matvec_w4a16_allreduce(x: *const CVoid, x_dtype: i32, awq: *const f32, mat: *const NveB200W4Matrix,
                                           k: i32, out_dtype: i32, stream: Stream) -> i32;
}

/// Turn a library status into a candle error (0 = ok).
fn b200_check(what: &str, status: i32) -> Result<()> {
    if status == 0 {
        Ok(())
    } else {
        candle_core::bail!("{}: libnve_kernels status {} (cudaError {})", what, status, unsafe { nve_b200_last_cuda_error() })
    }
}

/// RMSNorm + int8 quantise + q/k/v W4A8 GEMVs in one launch: replaces `apply_norm_gpu` + `quantize_f16_q8` +
/// three `matvec_w4a8` calls (src/gpu_layer.rs:1032-1038, 656-662).  `h`, `norm_w`: F16; weights as `GpuW4` fields.
pub fn rmsnorm_qkv_w4a8(
    h: &Tensor, norm_w: &Tensor, eps: f32,
    mats: &[(&Tensor, &Tensor, usize)], // (nibbles, scales, n) for q, k, v
    k: usize,
) -> Result<Vec<Tensor>> {
    let outs: Vec<Tensor> = mats.iter().map(|m| Tensor::zeros((1, m.2), DType::F16, h.device())).collect::<Result<_>>()?;
    let mut descs = Vec::with_capacity(mats.len());
    for (m, o) in mats.iter().zip(outs.iter()) {
        descs.push(NveB200W4Matrix {
            nibbles: cuda_dev_ptr_u8(m.0)? as *const u8,
            scales: cuda_dev_ptr_f32(m.1)? as *const f32,
            out: cuda_dev_ptr(o)? as *mut CVoid,
            residual: std::ptr::null(),
            n: m.2 as i32,
        });
    }
    let st = unsafe {
        nve_b200_rmsnorm_matvec_w4a8_multi(cuda_dev_ptr(h)? as *const CVoid, cuda_dev_ptr(norm_w)? as *const CVoid, eps,
                                           NVE_DT_F16, descs.as_ptr(), descs.len() as i32, k as i32, NVE_DT_F16, stream())
    };
    b200_check("nve_b200_rmsnorm_matvec_w4a8_multi", st)?;
    Ok(outs)
}

/// Batch > 1 branch of `GpuWeight::matmul_x` (src/gpu_layer.rs:235-237) without the dequantised copy: `x` [M, K] F16,
/// M <= 64 per call.  No workspace is allocated (the library's fixed 4 MiB array holds the split-K partial sums).
pub fn gemm_w4a16_noalloc(x: &Tensor, nibbles: &Tensor, scales: &Tensor, n: usize, k: usize) -> Result<Tensor> {
    let m = x.dim(0)?;
    let y = Tensor::zeros((m, n), DType::F16, x.device())?;
    let st = unsafe {
        nve_b200_gemm_w4a16_noalloc(cuda_dev_ptr(x)? as *const CVoid, NVE_DT_F16, cuda_dev_ptr_u8(nibbles)? as *const u8,
                                    cuda_dev_ptr_f32(scales)? as *const f32, cuda_dev_ptr(&y)? as *mut CVoid, NVE_DT_F16,
                                    m as i32, n as i32, k as i32, stream())
    };
    b200_check("nve_b200_gemm_w4a16_noalloc", st)?;
    Ok(y)
}
