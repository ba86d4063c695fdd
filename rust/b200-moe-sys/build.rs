// Links the prebuilt CUDA library.  mlx-sys builds its C++ dependency with cmake and runs bindgen
// (mlx-sys/build.rs); this crate does neither: libb200moe.so is built by nvcc outside cargo
// (`python mlx-rs_b200/build.py`) and src/lib.rs is generated from the header by gen_bindings.py.
use std::env;

fn main() {
    println!("cargo:rerun-if-env-changed=B200_MOE_LIB_DIR");
    println!("cargo:rerun-if-changed=../../include/b200_moe.h");
    let dir = env::var("B200_MOE_LIB_DIR")
        .expect("set B200_MOE_LIB_DIR to the directory that holds libb200moe.so");
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=b200moe");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
}
