//! `impl WeightAccel for CudaWeightAccel` (crates/strix-core/src/accel.rs:147-507): every hot-path method of the
//! trait forwarded to the C ABI; everything else keeps the trait's declining defaults. Uncompiled here.
use std::collections::HashMap;
use std::ffi::{CStr, CString};
use std::os::raw::c_char;

use strix_core::accel::{GpuDecodeConfig, WeightAccel};

use crate::ffi;

pub struct CudaWeightAccel {
    h: *mut ffi::StrixCuda,
    name: String,
    int8_act: bool,
    vocab: usize,
    moe_hidden: HashMap<usize, usize>,  // adopted mixture-of-experts layers -> hidden size (the length of their outputs)
}
// Same soundness argument as RocmWeightAccel (decode.rs:559-562): one caller at a time.
unsafe impl Send for CudaWeightAccel {}
unsafe impl Sync for CudaWeightAccel {}

fn cstr(p: *const c_char) -> String {
    if p.is_null() { String::new() } else { unsafe { CStr::from_ptr(p) }.to_string_lossy().into_owned() }
}

impl CudaWeightAccel {
    /// One accelerator on `device`; `rank` of `world` adopts its row shard of every uploaded weight.
    pub fn new(device: i32, rank: i32, world: i32) -> Result<Self, String> {
        let opts = ffi::StrixCudaOpts { rank, world, ..Default::default() };
        let mut h = std::ptr::null_mut();
        if unsafe { ffi::strix_cuda_create(device, &opts, &mut h) } != 1 {
            return Err(cstr(unsafe { ffi::strix_cuda_create_error() }));
        }
        let name = cstr(unsafe { ffi::strix_cuda_name(h) });
        // STRIX_NO_INT8 keeps the f32-activation kernels, as in decode.rs:771
        Ok(Self { h, name, int8_act: std::env::var("STRIX_NO_INT8").is_err(), vocab: 0, moe_hidden: HashMap::new() })
    }
    fn act(&self) -> i32 { if self.int8_act { ffi::ACT_Q8DOT } else { ffi::ACT_F32 } }
    fn rows(&self, key: &CString) -> Option<usize> {
        let (mut k, mut n, mut r0, mut rows, mut ty) = (0usize, 0usize, 0usize, 0usize, 0i32);
        (unsafe { ffi::strix_cuda_weight_info(self.h, key.as_ptr(), &mut k, &mut n, &mut r0, &mut rows, &mut ty) } == 1)
            .then_some(rows)
    }
    pub fn last_error(&self) -> String { cstr(unsafe { ffi::strix_cuda_last_error(self.h) }) }
}

macro_rules! upload {
    ($name:ident, $ffi:ident) => {
        fn $name(&mut self, key: &str, bytes: &[u8], in_dim: usize, out_dim: usize) -> bool {
            let k = match CString::new(key) { Ok(k) => k, Err(_) => return false };
            // `bytes` is borrowed for the call only: the library has copied it when this returns
            unsafe { ffi::$ffi(self.h, k.as_ptr(), bytes.as_ptr(), bytes.len(), in_dim, out_dim) == 1 }
        }
    };
}

impl WeightAccel for CudaWeightAccel {
    upload!(upload_q4_0, strix_cuda_upload_q4_0);
    upload!(upload_q4_1, strix_cuda_upload_q4_1);
    upload!(upload_q6_k, strix_cuda_upload_q6_k);
    upload!(upload_q8_0, strix_cuda_upload_q8_0);

    fn upload_f32(&mut self, key: &str, data: &[f32]) {
        if let Ok(k) = CString::new(key) {
            unsafe { ffi::strix_cuda_upload_f32(self.h, k.as_ptr(), data.as_ptr(), data.len()) };
        }
    }

    fn gemv(&self, key: &str, x: &[f32]) -> Option<Vec<f32>> {
        let k = CString::new(key).ok()?;
        let mut y = vec![0f32; self.rows(&k)?];
        let rc = unsafe { ffi::strix_cuda_gemv(self.h, k.as_ptr(), x.as_ptr(), x.len(), y.as_mut_ptr(), y.len(), self.act()) };
        (rc == 1).then_some(y) // 0 => None => the caller's CPU qmatmul (qwen3.rs:779-787)
    }

    fn gemv_batch(&self, calls: &[(&str, &[f32])]) -> Option<Vec<Vec<f32>>> {
        let keys: Vec<CString> = calls.iter().map(|(k, _)| CString::new(*k).ok()).collect::<Option<_>>()?;
        let kp: Vec<*const c_char> = keys.iter().map(|k| k.as_ptr()).collect();
        let xs: Vec<*const f32> = calls.iter().map(|(_, x)| x.as_ptr()).collect();
        let ks: Vec<usize> = calls.iter().map(|(_, x)| x.len()).collect();
        let mut ys: Vec<Vec<f32>> = keys.iter().map(|k| vec![0f32; self.rows(k).unwrap_or(0)]).collect();
        let yp: Vec<*mut f32> = ys.iter_mut().map(|y| y.as_mut_ptr()).collect();
        let caps: Vec<usize> = ys.iter().map(|y| y.len()).collect();
        let mut status = vec![0i32; calls.len()];
        let rc = unsafe {
            ffi::strix_cuda_gemv_batch(self.h, calls.len(), kp.as_ptr(), xs.as_ptr(), ks.as_ptr(), yp.as_ptr(), caps.as_ptr(),
                                       self.act(), status.as_mut_ptr())
        };
        (rc == 1 && status.iter().all(|s| *s == 1)).then_some(ys)
    }

    fn prefill_q8_gemm(&self, key: &str, xs: &[f32], m: usize) -> Option<Vec<f32>> {
        let k = CString::new(key).ok()?;
        let mut y = vec![0f32; m * self.rows(&k)?];
        let rc = unsafe { ffi::strix_cuda_prefill_q8_gemm(self.h, k.as_ptr(), xs.as_ptr(), m, y.as_mut_ptr(), y.len()) };
        (rc == 1).then_some(y)
    }

    // mixture-of-experts layers (accel.rs:167-246): whole-layer uploads, one token's routed FFN, grouped tokens
    fn upload_moe_q8(&mut self, layer: usize, gate: &[u8], up: &[u8], down: &[u8], hidden: usize, eff: usize, ne: usize) -> bool {
        let rc = unsafe {
            ffi::strix_cuda_upload_moe_q8(self.h, layer, gate.as_ptr(), gate.len(), up.as_ptr(), up.len(), down.as_ptr(),
                                          down.len(), hidden, eff, ne)
        };
        if rc == 1 { self.moe_hidden.insert(layer, hidden); }
        rc == 1
    }
    fn upload_moe_q6(&mut self, layer: usize, gate: &[u8], up: &[u8], down: &[u8], hidden: usize, eff: usize, ne: usize) -> bool {
        let rc = unsafe {
            ffi::strix_cuda_upload_moe_q6(self.h, layer, gate.as_ptr(), gate.len(), up.as_ptr(), up.len(), down.as_ptr(),
                                          down.len(), hidden, eff, ne)
        };
        if rc == 1 { self.moe_hidden.insert(layer, hidden); }
        rc == 1
    }
    fn moe_ffn(&self, layer: usize, ids: &[i32], wexp: &[f32], x: &[f32], sgate: f32) -> Option<Vec<f32>> {
        if ids.len() != wexp.len() { return None; }
        let mut y = vec![0f32; *self.moe_hidden.get(&layer)?];
        let rc = unsafe {
            ffi::strix_cuda_moe_ffn(self.h, layer, ids.as_ptr(), wexp.as_ptr(), ids.len(), x.as_ptr(), x.len(), sgate, self.act(),
                                    y.as_mut_ptr(), y.len())
        };
        (rc == 1).then_some(y)
    }
    fn moe_expert_ffn(&self, layer: usize, e: usize, xs: &[f32], m: usize) -> Option<Vec<f32>> {
        let mut y = vec![0f32; m * *self.moe_hidden.get(&layer)?];
        let rc = unsafe { ffi::strix_cuda_moe_expert_ffn(self.h, layer, e, xs.as_ptr(), m, self.act(), y.as_mut_ptr(), y.len()) };
        (rc == 1).then_some(y)
    }
    fn moe_layer_ffn(&self, layer: usize, plan: &[(i32, i32)], xs: &[f32], rows: usize) -> Option<Vec<f32>> {
        // (expert id, row count) pairs are two consecutive ints, which is what the C side reads
        let flat: Vec<i32> = plan.iter().flat_map(|(e, n)| [*e, *n]).collect();
        let mut y = vec![0f32; rows * *self.moe_hidden.get(&layer)?];
        let rc = unsafe {
            ffi::strix_cuda_moe_layer_ffn(self.h, layer, flat.as_ptr(), plan.len(), xs.as_ptr(), rows, self.act(), y.as_mut_ptr(),
                                          y.len())
        };
        (rc == 1).then_some(y)
    }

    fn lm_head_argmax_rows(&self, key: &str, xs: &[f32], m: usize) -> Option<Vec<u32>> {
        let k = CString::new(key).ok()?;
        let mut ids = vec![0u32; m];
        let rc = unsafe {
            ffi::strix_cuda_lm_head_argmax_rows(self.h, k.as_ptr(), xs.as_ptr(), xs.len(), m, self.act(), ids.as_mut_ptr(),
                                                std::ptr::null_mut())
        };
        (rc == 1).then_some(ids) // 0 => None: unknown key, xs.len() != m * in_dim, or m > 16 (decode.rs:3633-3635)
    }

    fn configure_decode(&mut self, c: GpuDecodeConfig) -> bool {
        // field-for-field copy of GpuDecodeConfig / GpuLayerCfg (accel.rs:19-72) into the plain-data mirror;
        // attn_standin_q = 0 asks for real attention (accepted for the dense Qwen3 flavour, declined otherwise)
        let layers: Vec<ffi::StrixGpuLayerCfg> = c.layers.iter().map(|l| ffi::StrixGpuLayerCfg {
            head_dim: l.head_dim as u32, n_kv: l.n_kv as u32, k_eq_v: l.k_eq_v as i32, rope_theta: l.rope_theta,
            is_local: l.is_local as i32, output_scale: l.output_scale, no_rope: l.no_rope as i32, rope_norm: l.rope_norm as i32,
        }).collect();
        let cfg = ffi::StrixGpuDecodeConfig {
            hidden: c.hidden as u32, n_heads: c.n_heads as u32, ffn: c.ffn as u32, vocab: c.vocab as u32,
            n_layers: c.n_layers as u32, eps: c.eps, final_softcap: c.final_softcap,
            attn_rsqrt: c.attn_rsqrt as i32, norm_v: c.norm_v as i32, qk_norm: c.qk_norm as i32,
            post_norm: c.post_norm as i32, act_gelu: c.act_gelu as i32, gpu_prefill: c.gpu_prefill as i32,
            n_swa: c.n_swa as u32, max_seq: c.max_seq as u32, layers: layers.as_ptr(),
            attn_standin_q: 0, act: self.act(),
        };
        self.vocab = c.vocab;
        unsafe { ffi::strix_cuda_configure_decode(self.h, &cfg) == 1 }
    }

    fn seed_decode_kv(&mut self, il: usize, k: &[f32], v: &[f32], tokens: usize) -> bool {
        unsafe { ffi::strix_cuda_seed_decode_kv(self.h, il, k.as_ptr(), v.as_ptr(), tokens) == 1 }
    }

    fn decode_step(&mut self, h: &[f32], pos: usize) -> Option<Vec<f32>> {
        let mut logits = vec![0f32; self.vocab];
        (unsafe { ffi::strix_cuda_decode_step(self.h, h.as_ptr(), pos, logits.as_mut_ptr(), logits.len()) } == 1).then_some(logits)
    }

    fn decode_step_argmax(&mut self, h: &[f32], pos: usize) -> Option<u32> {
        let mut id = 0u32;
        (unsafe { ffi::strix_cuda_decode_step_argmax(self.h, h.as_ptr(), pos, &mut id) } == 1).then_some(id)
    }

    fn prefill(&mut self, h: &[f32], start_pos: usize, m: usize) -> Option<Vec<f32>> {
        let mut logits = vec![0f32; self.vocab];
        (unsafe { ffi::strix_cuda_prefill(self.h, h.as_ptr(), start_pos, m, logits.as_mut_ptr(), logits.len()) } == 1)
            .then_some(logits)
    }

    fn prefill_max(&self) -> usize { unsafe { ffi::strix_cuda_prefill_max(self.h) } }

    fn verify(&mut self, h: &[f32], start_pos: usize, m: usize) -> Option<Vec<f32>> {
        let mut logits = vec![0f32; m * self.vocab];
        (unsafe { ffi::strix_cuda_verify(self.h, h.as_ptr(), start_pos, m, logits.as_mut_ptr(), logits.len()) } == 1)
            .then_some(logits)
    }

    fn resident_count(&self) -> usize { unsafe { ffi::strix_cuda_resident_count(self.h) } }
    fn name(&self) -> &str { &self.name }
}

impl Drop for CudaWeightAccel {
    fn drop(&mut self) { unsafe { ffi::strix_cuda_destroy(self.h) } }
}
