//! Safe wrappers over `ingot-cuda-sys` with the names and argument meaning of the reference's Metal boundary
//! (`Gpu`, `Buffer`, `Weight`, `Tensor`: src/metal.rs, src/metal_generic.rs, src/weights.rs), so that
//! `generic.rs` can hold either backend behind the same calls.  Only the one-device decode path is wrapped
//! here; groups, chains and the GGUF reader follow the same pattern (a handle, a status, `last_error`).
use ingot_cuda_sys as sys;
use std::ffi::CStr;
use std::io;
use std::ptr;
use std::rc::Rc;

pub type Result<T> = io::Result<T>;

fn invalid(msg: impl Into<String>) -> io::Error {
    io::Error::new(io::ErrorKind::InvalidData, msg.into())
}

struct Handle(*mut sys::ingot_gpu);
impl Drop for Handle {
    fn drop(&mut self) {
        // SAFETY: the handle came from ingot_gpu_create and is destroyed once.
        unsafe { sys::ingot_gpu_destroy(self.0) }
    }
}

/// One CUDA device (the reference's `Gpu`, src/metal.rs:193-208).
#[derive(Clone)]
pub struct Gpu(Rc<Handle>);

/// A device allocation owned by this value (the reference's `Buffer`).
pub struct Buffer {
    gpu: Gpu,
    ptr: *mut core::ffi::c_void,
    pooled: bool,
    pub bytes: usize,
}
impl Drop for Buffer {
    fn drop(&mut self) {
        // SAFETY: the pointer came from this handle's allocator and is released once.
        unsafe {
            if self.pooled {
                sys::ingot_output_release(self.gpu.raw(), self.ptr.cast());
            } else {
                sys::ingot_buffer_free(self.gpu.raw(), self.ptr);
            }
        }
    }
}

/// Tensor (src/gguf.rs:18-25) as the projections need it.
#[derive(Clone, Copy, Debug)]
pub struct Tensor {
    pub cols: u32,
    pub rows: u32,
    pub count: u32,
    pub kind: u32,
    pub stride: u32,
}

/// Weight (src/weights.rs:10-13): a resident matrix and its descriptor.
pub struct Weight {
    pub buffer: Buffer,
    pub tensor: Tensor,
}

impl Gpu {
    pub fn new(device: i32) -> Result<Self> {
        let mut h = ptr::null_mut();
        // SAFETY: `h` is a valid out-pointer.
        let st = unsafe { sys::ingot_gpu_create(device, &mut h) };
        if st != sys::INGOT_OK || h.is_null() {
            return Err(io::Error::other("no usable CUDA device"));
        }
        Ok(Self(Rc::new(Handle(h))))
    }
    fn raw(&self) -> *mut sys::ingot_gpu {
        self.0 .0
    }
    /// Status -> io::Error with the reference's error kinds (src/lib.rs:39-41).
    fn check(&self, st: sys::ingot_status) -> Result<()> {
        if st == sys::INGOT_OK {
            return Ok(());
        }
        // SAFETY: the library returns a NUL-terminated string that lives until the next call on this handle.
        let msg = unsafe { CStr::from_ptr(sys::ingot_last_error(self.raw())) }.to_string_lossy().into_owned();
        Err(match st {
            sys::INGOT_INVALID | sys::INGOT_UNSUPPORTED => invalid(msg),
            sys::INGOT_EOF => io::Error::new(io::ErrorKind::UnexpectedEof, msg),
            sys::INGOT_INTERRUPTED => io::Error::new(io::ErrorKind::Interrupted, msg),
            sys::INGOT_TIMEOUT => io::Error::new(io::ErrorKind::TimedOut, msg),
            _ => io::Error::other(msg),
        })
    }
    /// Gpu::configure_workspace (src/metal.rs:1335-1337).
    pub fn configure_workspace(&self, limit: usize) {
        // SAFETY: plain call on a live handle.
        let _ = unsafe { sys::ingot_gpu_configure_workspace(self.raw(), limit) };
    }
    /// Gpu::output (src/metal.rs:1278-1333).
    pub fn output(&self, count: usize) -> Result<Buffer> {
        let mut p: *mut f32 = ptr::null_mut();
        // SAFETY: `p` is a valid out-pointer.
        self.check(unsafe { sys::ingot_output_alloc(self.raw(), count, &mut p) })?;
        Ok(Buffer { gpu: self.clone(), ptr: p.cast(), pooled: true, bytes: count * 4 })
    }
    /// Gpu::floats (src/metal.rs:1270-1276).
    pub fn floats(&self, values: &[f32]) -> Result<Buffer> {
        let bytes = std::mem::size_of_val(values);
        let mut p = ptr::null_mut();
        // SAFETY: out-pointer valid; the upload copies `bytes` bytes from a live slice before returning.
        unsafe {
            self.check(sys::ingot_buffer_alloc(self.raw(), bytes, &mut p))?;
            let b = Buffer { gpu: self.clone(), ptr: p, pooled: false, bytes };
            self.check(sys::ingot_buffer_upload(self.raw(), p, values.as_ptr().cast(), bytes))?;
            self.check(sys::ingot_synchronize(self.raw()))?;
            Ok(b)
        }
    }
    /// Gpu::load_weight (src/metal.rs:546-582): validates the layout (kind, dims against the byte count) and makes the matrix resident.
    pub fn load_weight(&self, data: &[u8], t: Tensor) -> Result<Weight> {
        let mut p = ptr::null_mut();
        // SAFETY: the library copies `data` before returning and validates (kind, dims, stride) against its length.
        self.check(unsafe {
            sys::ingot_weight_upload(self.raw(), data.as_ptr().cast(), t.kind, t.cols as u64, t.rows as u64, t.count as u64,
                                     data.len(), &mut p)
        })?;
        Ok(Weight { buffer: Buffer { gpu: self.clone(), ptr: p, pooled: false, bytes: data.len() }, tensor: t })
    }
    /// Weight::matvec / Gpu::generic_project (src/weights.rs:142-186, src/metal_generic.rs:182-206): `count`
    /// rows of float32 activations against expert `expert` of the weight; more than four rows take the GEMM.
    pub fn matmul(&self, w: &Weight, expert: u32, x: &Buffer, count: u32) -> Result<Buffer> {
        let t = w.tensor;
        if expert >= t.count || x.bytes != 4 * t.cols as usize * count as usize {
            return Err(invalid("quantized dimensions mismatch"));
        }
        let y = self.output(t.rows as usize * count as usize)?;
        // SAFETY: all pointers are live device allocations of the checked sizes.
        self.check(unsafe {
            sys::ingot_matmul(self.raw(), w.buffer.ptr, t.cols, t.rows, t.stride, t.kind, expert, x.ptr, sys::INGOT_KIND_F32, count,
                              y.ptr.cast())
        })?;
        Ok(y)
    }
    /// Gpu::read_f32 after Gpu::complete (src/metal.rs:700-760): waits for the stream, copies to the host.
    pub fn read_f32(&self, b: &Buffer) -> Result<Vec<f32>> {
        let mut out = vec![0f32; b.bytes / 4];
        // SAFETY: `out` holds b.bytes bytes.
        self.check(unsafe { sys::ingot_buffer_read(self.raw(), out.as_mut_ptr().cast(), b.ptr, b.bytes) })?;
        if out.iter().any(|v| !v.is_finite()) {
            return Err(invalid("output contains non-finite values"));
        }
        Ok(out)
    }
}
