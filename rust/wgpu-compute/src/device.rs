//! `Device` (original: `src/device.rs:8-52`): a reference-counted handle on one GPU and its stream.
use crate::error::{check, Error};
use std::ptr;

pub struct Device {
    pub(crate) raw: *mut wgf_sys::wgf_device,
}

// The C ABI makes the device and its allocator thread-safe (one stream per device handle); user
// code of the original crate moves a clone into its poll thread.
unsafe impl Send for Device {}
unsafe impl Sync for Device {}

impl Clone for Device {
    fn clone(&self) -> Self {
        unsafe { wgf_sys::wgf_device_retain(self.raw) };
        Device { raw: self.raw }
    }
}

impl Drop for Device {
    fn drop(&mut self) {
        unsafe { wgf_sys::wgf_device_release(self.raw) };
    }
}

impl Device {
    /// GPU 0.  `async` only because the original is (`src/device.rs:14-32`): nothing is awaited.
    pub async fn new() -> Result<Self, Error> {
        Self::with_ordinal(0)
    }

    /// GPU `ordinal`; -1 is the compile-only device (resolves graphs and compiles kernels, runs nothing).
    pub fn with_ordinal(ordinal: i32) -> Result<Self, Error> {
        let mut raw = ptr::null_mut();
        check(unsafe { wgf_sys::wgf_device_create(ordinal, &mut raw) })?;
        Ok(Device { raw })
    }

    /// Kept so that `device.wgpu_device().poll(wgpu::PollType::Wait).unwrap()` still compiles
    /// (`src/device.rs:46`): the returned value only polls, and polling does nothing.
    pub fn wgpu_device(&self) -> &Self {
        self
    }

    /// No-op (`wgf_device_poll`).  Sleeps a little so that the usual `loop { poll }` thread does not spin.
    pub fn poll(&self, _how: crate::wgpu::PollType) -> Result<(), Error> {
        check(unsafe { wgf_sys::wgf_device_poll(self.raw) })?;
        std::thread::sleep(std::time::Duration::from_millis(50));
        Ok(())
    }

    /// Waits for everything queued on the device's stream.
    pub fn sync(&self) -> Result<(), Error> {
        check(unsafe { wgf_sys::wgf_device_sync(self.raw) })
    }

    /// Per-kernel event timing on / off (on by default, like the original's timestamp queries).
    pub fn set_timing(&self, enabled: bool) -> Result<(), Error> {
        check(unsafe { wgf_sys::wgf_device_set_timing(self.raw, enabled as i32) })
    }

    /// Kernels launched on this device so far.
    pub fn launch_count(&self) -> u64 {
        let mut n = 0u64;
        unsafe { wgf_sys::wgf_device_launch_count(self.raw, &mut n) };
        n
    }

    /// (bytes held from the driver, bytes handed out to live buffers)
    pub fn memory(&self) -> (u64, u64) {
        let (mut reserved, mut in_use) = (0u64, 0u64);
        unsafe { wgf_sys::wgf_device_memory(self.raw, &mut reserved, &mut in_use) };
        (reserved, in_use)
    }
}
