// Forwarding of the reference's kernel trait onto libmcb.so: what replaces the bodies of
// `impl Ops<CudaBackend> for CudaOps` in crates/modern-chainer-cuda/src/ops.rs:600-1925.  The trait
// (crates/modern-chainer-core/src/storage.rs:31-414) and every signature stay as they are; only the
// implementation behind them changes.  Raw declarations: mcb_sys.rs (generated from mcb.h).
//
// Not compiled where this library is built (no Rust toolchain there).  tests/test_cabi_load.py checks
// mechanically that every mcb_* call below names a function of mcb.h with the same number of arguments.
//
// Storage: `CudaStorage` wraps a device pointer from mcb_alloc and returns it with mcb_free in Drop
// (replaces CudaPool, src/backend.rs:13-107).  `CudaRuntime` holds the `*mut McbCtx`.
use std::ffi::CStr;
use std::sync::Arc;

use modern_chainer_core::{Activation, AdamConfig, Backend, DType, Error, Ops, Result, Shape, Tensor};

use crate::mcb_sys::*;
use crate::{CudaBackend, CudaRuntime, CudaStorage};

#[derive(Clone)]
pub struct CudaOps {
    pub(crate) runtime: Arc<CudaRuntime>,
}

fn dtype_code(dtype: DType) -> Result<i32> {
    Ok(match dtype {
        DType::F32 => MCB_F32,
        DType::I64 => MCB_I64,
        DType::I32 => MCB_I32,
        DType::U8 => MCB_U8,
        DType::F16 => MCB_F16,
        DType::BF16 => MCB_BF16,
        other => return Err(Error::UnsupportedDType(other)),
    })
}

impl CudaOps {
    fn ctx(&self) -> *mut McbCtx {
        self.runtime.ctx
    }

    fn message(&self) -> String {
        let p = unsafe { mcb_last_error(self.ctx()) };
        if p.is_null() {
            String::new()
        } else {
            unsafe { CStr::from_ptr(p) }.to_string_lossy().into_owned()
        }
    }

    /// mcb_status -> core::Error, one variant per code (crates/modern-chainer-core/src/error.rs:8-40).
    /// The structured variants carry the operands the caller still has in hand; the library's own message goes
    /// into the string-carrying ones.
    fn check(&self, status: Status, left: &Shape, right: &Shape, dtype: DType) -> Result<()> {
        match status {
            MCB_OK => Ok(()),
            MCB_SHAPE_MISMATCH => Err(Error::ShapeMismatch { context: self.message(), left: left.clone(), right: right.clone() }),
            MCB_BROADCAST => Err(Error::Broadcast { left: left.clone(), right: right.clone() }),
            MCB_DTYPE_MISMATCH => Err(Error::DTypeMismatch { expected: DType::F32, actual: dtype }),
            MCB_UNSUPPORTED_DTYPE => Err(Error::UnsupportedDType(dtype)),
            MCB_INVALID_ARGUMENT => Err(Error::InvalidArgument(self.message())),
            MCB_OUT_OF_BOUNDS => Err(Error::OutOfBounds { index: 0, len: left.numel() }),
            MCB_UNSUPPORTED => Err(Error::Unsupported(self.message())),
            MCB_IO => Err(Error::Io(std::io::Error::new(std::io::ErrorKind::Other, self.message()))),
            _ => Err(Error::Backend(format!("cuda {}", self.message()))), // MCB_BACKEND and anything unknown
        }
    }

    fn ok(&self, status: Status, t: &Tensor<CudaBackend>) -> Result<()> {
        self.check(status, t.shape(), t.shape(), t.dtype())
    }

    fn backend(&self) -> CudaBackend {
        CudaBackend { runtime: Arc::clone(&self.runtime), ops: self.clone() }
    }

    /// contiguous tensors only, as today (src/ops.rs:32-40); the offset is in elements
    fn ptr(&self, t: &Tensor<CudaBackend>) -> Result<*const core::ffi::c_void> {
        if !t.is_contiguous() {
            return Err(Error::InvalidArgument("cuda kernel requires a contiguous tensor".into()));
        }
        Ok(unsafe { t.storage().device_ptr().add(t.offset() * t.dtype().size_bytes()) } as *const _)
    }

    fn f32(&self, t: &Tensor<CudaBackend>) -> Result<*const f32> {
        if t.dtype() != DType::F32 {
            return Err(Error::UnsupportedDType(t.dtype()));
        }
        Ok(self.ptr(t)? as *const f32)
    }

    /// a new tensor whose storage comes from the library's caching allocator (not zero-filled: every
    /// kernel below writes all of its output)
    fn out(&self, shape: &Shape, dtype: DType) -> Result<Tensor<CudaBackend>> {
        let backend = self.backend();
        let storage = backend.alloc_for(shape.numel() * dtype.size_bytes(), dtype)?;
        Tensor::from_storage(backend, storage, shape.clone(), dtype)
    }

    fn dims(shape: &Shape) -> Vec<i64> {
        shape.dims().iter().map(|d| *d as i64).collect()
    }

    fn rows_and_last(t: &Tensor<CudaBackend>) -> Result<(i64, i64)> {
        let dims = t.shape().dims();
        let last = *dims.last().ok_or_else(|| Error::InvalidArgument("expected rank >= 1".into()))?;
        Ok(((t.numel() / last.max(1)) as i64, last as i64))
    }

    fn binary(&self, op: i32, a: &Tensor<CudaBackend>, b: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let shape = a.shape().broadcast_with(b.shape())?;
        let out = self.out(&shape, DType::F32)?;
        let (ad, bd) = (Self::dims(a.shape()), Self::dims(b.shape()));
        let st = unsafe {
            mcb_binary(self.ctx(), op, self.f32(a)?, ad.as_ptr(), ad.len() as i32, self.f32(b)?, bd.as_ptr(), bd.len() as i32, self.f32(&out)? as *mut f32)
        };
        self.check(st, a.shape(), b.shape(), a.dtype())?;
        Ok(out)
    }

    fn unary(&self, op: i32, x: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let out = self.out(x.shape(), DType::F32)?;
        let st = unsafe { mcb_unary(self.ctx(), op, self.f32(x)?, self.f32(&out)? as *mut f32, x.numel() as i64) };
        self.ok(st, x)?;
        Ok(out)
    }
}

impl Ops<CudaBackend> for CudaOps {
    fn add(&self, a: &Tensor<CudaBackend>, b: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.binary(MCB_ADD, a, b)
    }
    fn sub(&self, a: &Tensor<CudaBackend>, b: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.binary(MCB_SUB, a, b)
    }
    fn mul(&self, a: &Tensor<CudaBackend>, b: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.binary(MCB_MUL, a, b)
    }
    fn div(&self, a: &Tensor<CudaBackend>, b: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.binary(MCB_DIV, a, b)
    }
    fn sqrt(&self, a: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.unary(MCB_SQRT, a)
    }
    fn exp(&self, a: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.unary(MCB_EXP, a)
    }
    fn log(&self, a: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.unary(MCB_LOG, a)
    }
    fn sigmoid(&self, a: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.unary(MCB_SIGMOID, a)
    }
    fn silu(&self, a: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.unary(MCB_SILU, a)
    }
    fn abs(&self, a: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.unary(MCB_ABS, a)
    }

    fn relu(&self, x: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let out = self.out(x.shape(), x.dtype())?;
        let st = unsafe { mcb_relu(self.ctx(), self.ptr(x)?, self.ptr(&out)? as *mut _, x.numel() as i64, dtype_code(x.dtype())?) };
        self.ok(st, x)?;
        Ok(out)
    }
    fn relu_backward(&self, x: &Tensor<CudaBackend>, grad: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let out = self.out(x.shape(), x.dtype())?;
        let st = unsafe {
            mcb_relu_backward(self.ctx(), self.ptr(x)?, self.ptr(grad)?, self.ptr(&out)? as *mut _, x.numel() as i64, dtype_code(x.dtype())?)
        };
        self.ok(st, x)?;
        Ok(out)
    }
    fn gelu(&self, x: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let out = self.out(x.shape(), x.dtype())?;
        let st = unsafe { mcb_gelu(self.ctx(), self.ptr(x)?, self.ptr(&out)? as *mut _, x.numel() as i64, dtype_code(x.dtype())?) };
        self.ok(st, x)?;
        Ok(out)
    }

    fn matmul(&self, a: &Tensor<CudaBackend>, b: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let (ad, bd) = (a.shape().dims(), b.shape().dims());
        if ad.len() != 2 || bd.len() != 2 || ad[1] != bd[0] {
            return Err(Error::ShapeMismatch { context: "matmul".into(), left: a.shape().clone(), right: b.shape().clone() });
        }
        let out = self.out(&Shape::new(vec![ad[0], bd[1]]), DType::F32)?;
        let st = unsafe { mcb_matmul(self.ctx(), self.f32(a)?, self.f32(b)?, self.f32(&out)? as *mut f32, ad[0] as i64, ad[1] as i64, bd[1] as i64) };
        self.check(st, a.shape(), b.shape(), a.dtype())?;
        Ok(out)
    }

    fn linear(&self, x: &Tensor<CudaBackend>, weight: &Tensor<CudaBackend>, bias: Option<&Tensor<CudaBackend>>) -> Result<Tensor<CudaBackend>> {
        self.linear_activation(x, weight, bias, Activation::None)
    }

    fn linear_activation(&self, x: &Tensor<CudaBackend>, weight: &Tensor<CudaBackend>, bias: Option<&Tensor<CudaBackend>>,
                         activation: Activation) -> Result<Tensor<CudaBackend>> {
        let (m, k) = Self::rows_and_last(x)?;
        let n = weight.shape().dims()[0] as i64;
        let mut dims = x.shape().dims().to_vec();
        *dims.last_mut().unwrap() = n as usize;
        let out = self.out(&Shape::new(dims), DType::F32)?;
        let act = match activation {
            Activation::None => MCB_ACT_NONE,
            Activation::Relu => MCB_ACT_RELU,
            Activation::Gelu => MCB_ACT_GELU,
            other => return Err(Error::Unsupported(format!("linear_activation({other:?})"))),
        };
        let b = match bias { Some(b) => self.f32(b)?, None => core::ptr::null() };
        // autocast / ComputeType are applied inside the library (mcb_set_autocast, mcb_set_compute_type)
        let st = unsafe { mcb_linear(self.ctx(), self.f32(x)?, self.f32(weight)?, b, self.f32(&out)? as *mut f32, m, k, n, act) };
        self.check(st, x.shape(), weight.shape(), x.dtype())?;
        Ok(out)
    }

    fn linear_backward(&self, grad: &Tensor<CudaBackend>, x: &Tensor<CudaBackend>, weight: &Tensor<CudaBackend>)
        -> Result<(Tensor<CudaBackend>, Tensor<CudaBackend>)> {
        let (m, k) = Self::rows_and_last(x)?;
        let n = weight.shape().dims()[0] as i64;
        let (dx, dw) = (self.out(x.shape(), DType::F32)?, self.out(weight.shape(), DType::F32)?);
        let st = unsafe {
            mcb_linear_backward(self.ctx(), self.f32(grad)?, self.f32(x)?, self.f32(weight)?, self.f32(&dx)? as *mut f32, self.f32(&dw)? as *mut f32,
                                core::ptr::null_mut(), m, k, n)
        };
        self.check(st, grad.shape(), weight.shape(), grad.dtype())?;
        Ok((dx, dw))
    }

    fn linear_backward_with_bias(&self, grad: &Tensor<CudaBackend>, x: &Tensor<CudaBackend>, weight: &Tensor<CudaBackend>, bias_shape: &Shape)
        -> Result<(Tensor<CudaBackend>, Tensor<CudaBackend>, Tensor<CudaBackend>)> {
        let (m, k) = Self::rows_and_last(x)?;
        let n = weight.shape().dims()[0] as i64;
        let (dx, dw, db) = (self.out(x.shape(), DType::F32)?, self.out(weight.shape(), DType::F32)?, self.out(bias_shape, DType::F32)?);
        let st = unsafe {
            mcb_linear_backward(self.ctx(), self.f32(grad)?, self.f32(x)?, self.f32(weight)?, self.f32(&dx)? as *mut f32, self.f32(&dw)? as *mut f32,
                                self.f32(&db)? as *mut f32, m, k, n)
        };
        self.check(st, grad.shape(), weight.shape(), grad.dtype())?;
        Ok((dx, dw, db))
    }

    fn transpose2d(&self, a: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let d = a.shape().dims();
        if d.len() != 2 {
            return Err(Error::InvalidArgument(format!("transpose2d expects a 2-D tensor, got rank {}", d.len())));
        }
        let out = self.out(&Shape::new(vec![d[1], d[0]]), DType::F32)?;
        let st = unsafe { mcb_transpose2d(self.ctx(), self.f32(a)?, self.f32(&out)? as *mut f32, d[0] as i64, d[1] as i64) };
        self.ok(st, a)?;
        Ok(out)
    }

    fn embedding(&self, ids: &Tensor<CudaBackend>, weight: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let wd = weight.shape().dims();
        let mut dims = ids.shape().dims().to_vec();
        dims.push(wd[1]);
        let out = self.out(&Shape::new(dims), DType::F32)?;
        let st = unsafe {
            mcb_embedding(self.ctx(), self.ptr(ids)?, dtype_code(ids.dtype())?, ids.numel() as i64, self.f32(weight)?, wd[0] as i64, wd[1] as i64,
                          self.f32(&out)? as *mut f32)
        };
        self.ok(st, ids)?;
        Ok(out)
    }

    fn embedding_backward(&self, ids: &Tensor<CudaBackend>, weight: &Tensor<CudaBackend>, grad: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let wd = weight.shape().dims();
        let out = self.out(weight.shape(), DType::F32)?;
        let st = unsafe {
            mcb_embedding_backward(self.ctx(), self.ptr(ids)?, dtype_code(ids.dtype())?, ids.numel() as i64, self.ptr(grad)?, dtype_code(grad.dtype())?,
                                   wd[0] as i64, wd[1] as i64, self.f32(&out)? as *mut f32, 0)
        };
        self.ok(st, ids)?;
        Ok(out)
    }

    fn layer_norm(&self, x: &Tensor<CudaBackend>, gamma: &Tensor<CudaBackend>, beta: &Tensor<CudaBackend>, eps: f64) -> Result<Tensor<CudaBackend>> {
        let (rows, dim) = Self::rows_and_last(x)?;
        let out = self.out(x.shape(), DType::F32)?;
        let st = unsafe {
            mcb_layer_norm(self.ctx(), self.f32(x)?, self.f32(gamma)?, self.f32(beta)?, eps, self.ptr(&out)? as *mut _, MCB_F32, core::ptr::null_mut(),
                           core::ptr::null_mut(), rows, dim)
        };
        self.check(st, x.shape(), gamma.shape(), x.dtype())?;
        Ok(out)
    }

    fn layer_norm_backward(&self, x: &Tensor<CudaBackend>, gamma: &Tensor<CudaBackend>, _beta: &Tensor<CudaBackend>, grad: &Tensor<CudaBackend>, eps: f64)
        -> Result<(Tensor<CudaBackend>, Tensor<CudaBackend>, Tensor<CudaBackend>)> {
        let (rows, dim) = Self::rows_and_last(x)?;
        let (dx, dg, db) = (self.out(x.shape(), DType::F32)?, self.out(gamma.shape(), DType::F32)?, self.out(gamma.shape(), DType::F32)?);
        let st = unsafe {
            mcb_layer_norm_backward(self.ctx(), self.f32(x)?, self.f32(gamma)?, self.ptr(grad)?, dtype_code(grad.dtype())?, eps, core::ptr::null(),
                                    core::ptr::null(), self.f32(&dx)? as *mut f32, self.f32(&dg)? as *mut f32, self.f32(&db)? as *mut f32, rows, dim)
        };
        self.check(st, x.shape(), grad.shape(), grad.dtype())?;
        Ok((dx, dg, db))
    }

    fn softmax_last_dim(&self, x: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let (rows, cols) = Self::rows_and_last(x)?;
        let out = self.out(x.shape(), DType::F32)?;
        let st = unsafe { mcb_softmax(self.ctx(), self.f32(x)?, self.f32(&out)? as *mut f32, rows, cols) };
        self.ok(st, x)?;
        Ok(out)
    }

    fn softmax_last_dim_backward(&self, x: &Tensor<CudaBackend>, grad: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let (rows, cols) = Self::rows_and_last(x)?;
        let out = self.out(x.shape(), DType::F32)?;
        let st = unsafe { mcb_softmax_backward(self.ctx(), self.f32(x)?, self.f32(grad)?, self.f32(&out)? as *mut f32, rows, cols) };
        self.check(st, x.shape(), grad.shape(), x.dtype())?;
        Ok(out)
    }

    fn softmax_cross_entropy(&self, logits: &Tensor<CudaBackend>, target: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let d = logits.shape().dims();
        let out = self.out(&Shape::scalar(), DType::F32)?;
        let st = unsafe {
            mcb_softmax_cross_entropy(self.ctx(), self.f32(logits)?, self.ptr(target)?, dtype_code(target.dtype())?, d[0] as i64, d[1] as i64,
                                      self.f32(&out)? as *mut f32)
        };
        self.check(st, logits.shape(), target.shape(), target.dtype())?;
        Ok(out)
    }

    fn softmax_cross_entropy_backward(&self, logits: &Tensor<CudaBackend>, target: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let d = logits.shape().dims();
        let out = self.out(logits.shape(), DType::F32)?;
        let st = unsafe {
            mcb_softmax_cross_entropy_backward(self.ctx(), self.f32(logits)?, self.ptr(target)?, dtype_code(target.dtype())?, d[0] as i64, d[1] as i64,
                                               self.f32(&out)? as *mut f32)
        };
        self.check(st, logits.shape(), target.shape(), target.dtype())?;
        Ok(out)
    }

    fn adam_update(&self, param: &Tensor<CudaBackend>, grad: &Tensor<CudaBackend>, m: &Tensor<CudaBackend>, v: &Tensor<CudaBackend>, cfg: &AdamConfig)
        -> Result<(Tensor<CudaBackend>, Tensor<CudaBackend>, Tensor<CudaBackend>)> {
        let (np, nm, nv) = (self.out(param.shape(), DType::F32)?, self.out(param.shape(), DType::F32)?, self.out(param.shape(), DType::F32)?);
        let st = unsafe {
            mcb_adam_update(self.ctx(), self.f32(param)?, self.f32(grad)?, self.f32(m)?, self.f32(v)?, self.f32(&np)? as *mut f32, self.f32(&nm)? as *mut f32,
                            self.f32(&nv)? as *mut f32, param.numel() as i64, cfg.lr, cfg.beta1, cfg.beta2, cfg.eps, cfg.step as i32)
        };
        self.check(st, param.shape(), grad.shape(), grad.dtype())?;
        Ok((np, nm, nv))
    }

    fn sum_all(&self, a: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        let out = self.out(&Shape::scalar(), DType::F32)?;
        let st = unsafe { mcb_sum_all(self.ctx(), self.f32(a)?, a.numel() as i64, self.f32(&out)? as *mut f32) };
        self.ok(st, a)?;
        Ok(out)
    }

    fn sum_to(&self, a: &Tensor<CudaBackend>, shape: &Shape) -> Result<Tensor<CudaBackend>> {
        let out = self.out(shape, DType::F32)?;
        let (ad, td) = (Self::dims(a.shape()), Self::dims(shape));
        let st = unsafe { mcb_sum_to(self.ctx(), self.f32(a)?, ad.as_ptr(), ad.len() as i32, td.as_ptr(), td.len() as i32, self.f32(&out)? as *mut f32) };
        self.check(st, a.shape(), shape, a.dtype())?;
        Ok(out)
    }

    fn scale(&self, a: &Tensor<CudaBackend>, factor: f64) -> Result<Tensor<CudaBackend>> {
        let out = self.out(a.shape(), DType::F32)?;
        let st = unsafe { mcb_scale(self.ctx(), self.f32(a)?, factor, self.f32(&out)? as *mut f32, a.numel() as i64) };
        self.ok(st, a)?;
        Ok(out)
    }

    fn full_like(&self, a: &Tensor<CudaBackend>, value: f64) -> Result<Tensor<CudaBackend>> {
        let out = self.out(a.shape(), DType::F32)?;
        let st = unsafe { mcb_fill(self.ctx(), self.f32(&out)? as *mut f32, value as f32, a.numel() as i64) };
        self.ok(st, a)?;
        Ok(out)
    }
    fn ones_like(&self, a: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.full_like(a, 1.0)
    }
    fn zeros_like(&self, a: &Tensor<CudaBackend>) -> Result<Tensor<CudaBackend>> {
        self.full_like(a, 0.0)
    }

    fn to_scalar(&self, a: &Tensor<CudaBackend>) -> Result<f64> {
        let mut host = 0f32;
        // synchronises; also the point where a label / index fault found on the device surfaces as InvalidArgument
        let st = unsafe { mcb_memcpy_d2h(self.ctx(), &mut host as *mut f32 as *mut _, self.ptr(a)?, 4) };
        self.ok(st, a)?;
        Ok(host as f64)
    }

    fn cast(&self, x: &Tensor<CudaBackend>, dtype: DType) -> Result<Tensor<CudaBackend>> {
        let out = self.out(x.shape(), dtype)?;
        let st = unsafe { mcb_cast(self.ctx(), self.ptr(x)?, dtype_code(x.dtype())?, self.ptr(&out)? as *mut _, dtype_code(dtype)?, x.numel() as i64) };
        self.ok(st, x)?;
        Ok(out)
    }

    fn attention(&self, q: &Tensor<CudaBackend>, k: &Tensor<CudaBackend>, v: &Tensor<CudaBackend>, heads: usize, causal: bool) -> Result<Tensor<CudaBackend>> {
        let d = q.shape().dims();
        let out = self.out(q.shape(), q.dtype())?;
        let st = unsafe {
            mcb_attention(self.ctx(), self.ptr(q)?, self.ptr(k)?, self.ptr(v)?, self.ptr(&out)? as *mut _, core::ptr::null_mut(), d[0] as i64, d[1] as i64,
                          d[2] as i64, heads as i64, causal as i32, dtype_code(q.dtype())?)
        };
        self.check(st, q.shape(), k.shape(), q.dtype())?;
        Ok(out)
    }
}
