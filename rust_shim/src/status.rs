//! Status code of `libkaio_b200.so` -> `KaioError`.
//!
//! NOT COMPILED IN THIS REPOSITORY: no Rust toolchain is available where it was written.
//!
//! `KaioError` (kaio-runtime/src/error.rs:4-37) keeps host-contract violations
//! (`InvalidConfig`), driver failures (`Cuda`) and target-capability failures (`Validation`)
//! apart, and callers match on them (the candle bridge prefixes and forwards the text,
//! kaio-candle/src/bridge.rs:176-178).  The mapping below keeps them apart too:
//!
//! | status | meaning                                   | `KaioError`                                   |
//! |--------|-------------------------------------------|-----------------------------------------------|
//! | 1      | argument contract violated                | `InvalidConfig(text)` -- the reference's text  |
//! | 2      | a CUDA runtime / driver call failed       | `Backend { code: 2, .. }` (`Cuda`-class)       |
//! | 3      | the device is not sm_100                  | `Validation(SmTooLow { .. })`                  |
//! | 4      | a device-side bounded wait gave up        | `Backend { code: 4, .. }`                      |
//!
//! `KaioError::Cuda` wraps a `cudarc::driver::DriverError`, which cannot be built from a
//! message, so statuses 2 and 4 need ONE additive variant in `kaio-runtime/src/error.rs`:
//!
//! ```ignore
//! /// The sm_100a backend library reported a failure that is not a contract violation.
//! #[error("kaio_b200 backend error {code}: {message}")]
//! Backend { code: i32, message: String },
//! ```

use std::ffi::CStr;

use kaio_core::ir::ValidationError;
use kaio_runtime::{KaioError, Result};

use crate::ffi;

/// Compute capability the backend library is built for (sm_100a).
const REQUIRED_SM: u32 = 100;

fn last_message() -> String {
    // SAFETY: the library returns a NUL-terminated string owned by the calling thread's state.
    unsafe { CStr::from_ptr(ffi::kaio_b200_last_error()) }
        .to_string_lossy()
        .into_owned()
}

/// Turn a status code into the reference's error type.  `actual_sm` is the device's compute
/// capability (major * 10 + minor), used only to fill `SmTooLow`.
pub fn check(code: i32, actual_sm: u32) -> Result<()> {
    match code {
        ffi::KAIO_B200_OK => Ok(()),
        ffi::KAIO_B200_ERR_INVALID_CONFIG => Err(KaioError::InvalidConfig(last_message())),
        ffi::KAIO_B200_ERR_UNSUPPORTED_ARCH => Err(KaioError::Validation(ValidationError::SmTooLow {
            required: REQUIRED_SM,
            actual: actual_sm,
            feature: "tcgen05.mma (libkaio_b200 is built for sm_100a)".to_string(),
        })),
        // 2 = CUDA error, 4 = device-side wait gave up, anything else = a newer library
        other => Err(KaioError::Backend { code: other, message: last_message() }),
    }
}
