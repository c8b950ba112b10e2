//! Kernel timing (original: `src/query.rs:10-126`).  The original wraps a wgpu timestamp query set
//! per kernel; here the library keeps a CUDA event pair per launch and reports nanoseconds.
use std::fmt;
use std::time::Duration;

/// Device time of one kernel launched while resolving a tensor's graph.
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub struct QueryResults {
    nanos: u64,
}

impl QueryResults {
    pub(crate) fn from_nanos(nanos: u64) -> Self {
        QueryResults { nanos }
    }

    pub fn elapsed(&self) -> Duration {
        Duration::from_nanos(self.nanos)
    }
}

impl fmt::Display for QueryResults {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        write!(f, "{:?}", self.elapsed())
    }
}

/// The original exports this type for its kernel-level API (`Option<&PerformanceQueries>`).  Its
/// counterpart in the C ABI is the `wgf_timing` handle a kernel-level launch hands back; this owns one.
pub struct PerformanceQueries {
    pub(crate) raw: *mut wgf_sys::wgf_timing,
}

impl PerformanceQueries {
    /// An empty query set for a kernel-level call to fill (`PerformanceQueries::new`,
    /// `src/query.rs:51-76`; the device argument is kept for the signature, the handle is created by
    /// the launch that receives `&mut self.raw`).  The wgpu-specific `resolve` and
    /// `compute_timestamp_writes` of the original have no counterpart: the library records its event
    /// pair inside the launch.
    pub fn new(_device: &crate::Device) -> Self {
        PerformanceQueries { raw: std::ptr::null_mut() }
    }

    /// Waits for the kernels of the call and returns their summed device time
    /// (`PerformanceQueries::wait_for_results`, `src/query.rs:78-112`).
    pub async fn wait_for_results(&self) -> QueryResults {
        let mut ns = 0u64;
        if !self.raw.is_null() {
            crate::error::expect(unsafe { wgf_sys::wgf_timing_elapsed_ns(self.raw, &mut ns) });
        }
        QueryResults::from_nanos(ns)
    }
}

impl Drop for PerformanceQueries {
    fn drop(&mut self) {
        if !self.raw.is_null() {
            unsafe { wgf_sys::wgf_timing_release(self.raw) };
        }
    }
}
