//! Modules of the routed block with the `forward` shape of `mlx_rs::module::Module`
//! (`mlx-rs/src/module/module.rs:27-44`; template `impl Module<&Array> for Mlp`,
//! `mlx-lm/src/models/qwen3.rs:204-255`).  Parameters keep the field names of `QuantizedLinear`
//! (`weight` / `scales` / `biases`, `group_size`, `bits`: `mlx-rs/src/nn/quantized.rs:307-335`), stacked over
//! the experts, and the projection names `gate_proj` / `up_proj` / `down_proj`.
use b200_moe_sys as sys;

use crate::buffer::{Context, DType, DeviceAllocator, DeviceBuf, Stream};
use crate::error::{guarded, Exception};

/// The trait the reference's modules implement, restated so that this crate stands alone; a host that links
/// `mlx-rs` implements its `Module` by forwarding to these.
pub trait Module<Input> {
    type Output;
    type Error;
    fn forward(&mut self, input: Input) -> Result<Self::Output, Self::Error>;
    fn training_mode(&mut self, mode: bool);
}

/// Stacked quantized projection of all experts: weight [E, out, in*bits/32] u32, scales / biases [E, out, in/gs] bf16.
pub struct QuantizedSwitchLinear<'a> {
    pub weight: DeviceBuf<'a>,
    pub scales: DeviceBuf<'a>,
    pub biases: DeviceBuf<'a>,
    pub group_size: i32,
    pub bits: i32,
}
impl QuantizedSwitchLinear<'_> {
    fn raw(&self) -> sys::b200_qlinear {
        sys::b200_qlinear { weight: self.weight.ptr as *const u32, scales: self.scales.ptr, biases: self.biases.ptr }
    }
}

/// `SwitchGlu::forward((x [.., H], indices [.., k])) -> [.., k, H]`.
pub struct SwitchGlu<'a> {
    pub gate_proj: QuantizedSwitchLinear<'a>,
    pub up_proj: QuantizedSwitchLinear<'a>,
    pub down_proj: QuantizedSwitchLinear<'a>,
    pub ctx: &'a Context,
    pub alloc: &'a dyn DeviceAllocator,
    pub stream: Stream,
}
impl<'a> SwitchGlu<'a> {
    fn dims(&self) -> (i32, i32, i32) {
        // gate_proj.weight [E, I, H*bits/32], down_proj.weight [E, H, I*bits/32]
        (self.down_proj.weight.dim(1) as i32, self.gate_proj.weight.dim(1) as i32, self.gate_proj.weight.dim(0) as i32)
    }
    fn config(&self, top_k: i32, router_mode: i32, norm_topk_prob: bool) -> sys::b200_moe_config {
        let (hidden, inter, n_experts) = self.dims();
        sys::b200_moe_config { hidden, inter, n_experts, top_k, bits: self.gate_proj.bits, group_size: self.gate_proj.group_size,
                               router_mode, norm_topk_prob: norm_topk_prob as i32 }
    }
    fn params(&self, router_weight: *const std::os::raw::c_void, bias: *const f32) -> sys::b200_moe_params {
        sys::b200_moe_params { router_weight, router_logit_bias: bias, gate_proj: self.gate_proj.raw(), up_proj: self.up_proj.raw(),
                               down_proj: self.down_proj.raw() }
    }
}
impl<'a, 'b> Module<(&'b DeviceBuf<'b>, &'b DeviceBuf<'b>)> for SwitchGlu<'a> {
    type Output = DeviceBuf<'a>;
    type Error = Exception;

    #[track_caller]
    fn forward(&mut self, (x, indices): (&'b DeviceBuf<'b>, &'b DeviceBuf<'b>)) -> Result<Self::Output, Self::Error> {
        let k = indices.dim(-1);
        let t = indices.numel() / k;
        let (hidden, _, _) = self.dims();
        let mut shape = indices.shape.clone();
        shape.push(hidden as i64);
        let out = DeviceBuf::new_in(self.alloc, DType::Bfloat16, &shape);
        let (cfg, params) = (self.config(k as i32, sys::B200_ROUTER_SOFTMAX_TOPK, true), self.params(std::ptr::null(), std::ptr::null()));
        guarded(|| unsafe {
            sys::b200_switch_glu_forward(self.ctx.raw, &cfg, &params, x.ptr, indices.ptr as *const u32, t, out.ptr, self.stream.0)
        })?;
        Ok(out)
    }

    fn training_mode(&mut self, _mode: bool) {}
}

/// `MoeBlock::forward(x [B, L, H]) -> [B, L, H]`: gate (router Linear, weight [E, H]) + switch_mlp.
pub struct MoeBlock<'a> {
    pub gate_weight: DeviceBuf<'a>,
    pub router_logit_bias: Option<DeviceBuf<'a>>,
    pub switch_mlp: SwitchGlu<'a>,
    pub top_k: i32,
    pub norm_topk_prob: bool,
    pub router_mode: i32,
}
impl<'a, 'b> Module<&'b DeviceBuf<'b>> for MoeBlock<'a> {
    type Output = DeviceBuf<'a>;
    type Error = Exception;

    #[track_caller]
    fn forward(&mut self, x: &'b DeviceBuf<'b>) -> Result<Self::Output, Self::Error> {
        let t = x.numel() / x.dim(-1);
        let mlp = &self.switch_mlp;
        let out = DeviceBuf::new_in(mlp.alloc, x.dtype, &x.shape);
        let cfg = mlp.config(self.top_k, self.router_mode, self.norm_topk_prob);
        let bias = self.router_logit_bias.as_ref().map_or(std::ptr::null(), |b| b.ptr as *const f32);
        let params = mlp.params(self.gate_weight.ptr, bias);
        guarded(|| unsafe {
            sys::b200_moe_block_forward(mlp.ctx.raw, &cfg, &params, x.ptr, t, out.ptr, std::ptr::null(), mlp.stream.0)
        })?;
        Ok(out)
    }

    fn training_mode(&mut self, _mode: bool) {}
}
