//! Status int -> message -> `Exception`, the convention of `mlx-rs/src/error.rs:226-280` and
//! `mlx-rs/src/utils/guard.rs:20-49`: the library calls the registered handler with the message, the handler
//! stores a copy in a thread-local, the wrapper turns a non-zero status into an `Exception`.
use std::cell::Cell;
use std::ffi::{c_void, CStr};
use std::os::raw::c_char;
use std::panic::Location;
use std::sync::Once;

/// What failed and where the failing op was called (same fields as `mlx_rs::error::Exception`).
#[derive(Debug, Clone, PartialEq)]
pub struct Exception {
    pub what: String,
    pub location: &'static Location<'static>,
}

impl std::fmt::Display for Exception {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "{} at {}:{}", self.what, self.location.file(), self.location.line())
    }
}
impl std::error::Error for Exception {}

thread_local! {
    static LAST_ERROR: Cell<*mut c_char> = const { Cell::new(std::ptr::null_mut()) };
}
static INIT_HANDLER: Once = Once::new();

extern "C" fn store_message(msg: *const c_char, _data: *mut c_void) {
    LAST_ERROR.with(|slot| {
        let old = slot.replace(unsafe { libc::strdup(msg) });
        if !old.is_null() {
            unsafe { libc::free(old as *mut libc::c_void) };
        }
    });
}
extern "C" fn no_dtor(_data: *mut c_void) {}

fn take_message() -> String {
    LAST_ERROR.with(|slot| {
        let p = slot.replace(std::ptr::null_mut());
        if p.is_null() {
            // the handler is process-wide but the slot is per thread: fall back to the library's own slot
            let q = unsafe { b200_moe_sys::b200_last_error() };
            return if q.is_null() { String::from("unknown error") } else { unsafe { CStr::from_ptr(q) }.to_string_lossy().into_owned() };
        }
        let s = unsafe { CStr::from_ptr(p) }.to_string_lossy().into_owned();
        unsafe { libc::free(p as *mut libc::c_void) };
        s
    })
}

/// Runs one library call and maps its status.
#[track_caller]
pub(crate) fn guarded<F: FnOnce() -> i32>(f: F) -> Result<(), Exception> {
    INIT_HANDLER.call_once(|| unsafe {
        b200_moe_sys::b200_set_error_handler(Some(store_message), std::ptr::null_mut(), Some(no_dtor));
    });
    match f() {
        0 => Ok(()),
        _ => Err(Exception { what: take_message(), location: Location::caller() }),
    }
}
