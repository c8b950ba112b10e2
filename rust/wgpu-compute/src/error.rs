//! Status codes of the C ABI as a Rust error.  (The original crate panics on shape and type misuse
//! and has two `Result`s: device creation and download.  The tensor-building methods here panic
//! with the library's message in the same situations; fallible entry points return `Error`.)
use std::ffi::CStr;
use std::fmt;

#[derive(Clone, Debug, PartialEq, Eq)]
pub struct Error {
    /// One of the `WGF_ERR_*` codes of `include/wgf.h`.
    pub code: i32,
    pub message: String,
}

impl fmt::Display for Error {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        write!(f, "{} ({})", self.message, self.name())
    }
}

impl std::error::Error for Error {}

impl Error {
    pub fn name(&self) -> &'static str {
        match self.code {
            wgf_sys::WGF_ERR_SHAPE => "WGF_ERR_SHAPE",
            wgf_sys::WGF_ERR_DTYPE => "WGF_ERR_DTYPE",
            wgf_sys::WGF_ERR_RANK => "WGF_ERR_RANK",
            wgf_sys::WGF_ERR_OOM => "WGF_ERR_OOM",
            wgf_sys::WGF_ERR_CUDA => "WGF_ERR_CUDA",
            wgf_sys::WGF_ERR_NCCL => "WGF_ERR_NCCL",
            wgf_sys::WGF_ERR_TIMEOUT => "WGF_ERR_TIMEOUT",
            wgf_sys::WGF_ERR_INVALID_HANDLE => "WGF_ERR_INVALID_HANDLE",
            wgf_sys::WGF_ERR_INVALID_ARGUMENT => "WGF_ERR_INVALID_ARGUMENT",
            wgf_sys::WGF_ERR_COMPILE => "WGF_ERR_COMPILE",
            wgf_sys::WGF_ERR_UNSUPPORTED => "WGF_ERR_UNSUPPORTED",
            _ => "WGF_ERR_?",
        }
    }
}

/// Turns a status into a `Result`, fetching the thread-local message on failure.
pub(crate) fn check(status: i32) -> Result<(), Error> {
    if status == wgf_sys::WGF_OK {
        return Ok(());
    }
    let message = unsafe {
        let p = wgf_sys::wgf_last_error();
        if p.is_null() {
            String::new()
        } else {
            CStr::from_ptr(p).to_string_lossy().into_owned()
        }
    };
    Err(Error { code: status, message })
}

/// For the graph-building calls, which the original crate makes infallible (it panics).
pub(crate) fn expect(status: i32) {
    if let Err(e) = check(status) {
        panic!("{e}");
    }
}
