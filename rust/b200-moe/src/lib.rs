//! Safe layer over `b200-moe-sys`, shaped like `mlx-rs`: op wrappers with the reference's names, argument
//! order and defaults (`ops`), and the module types of the routed block (`nn`).  UNVERIFIED (never compiled).
pub mod buffer;
pub mod error;
pub mod nn;
pub mod ops;

pub use buffer::{Context, DType, DeviceAllocator, DeviceBuf, Stream};
pub use error::Exception;

/// Result of every op, as in `mlx_rs::error::Result`.
pub type Result<T> = std::result::Result<T, Exception>;
