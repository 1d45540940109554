// UNCOMPILED IN THIS TREE (no Rust toolchain where the library is built).
//
// Points the linker at libtorchburn_b200.so.  TORCHBURN_B200_LIB_DIR names the directory that
// holds it (default: the in-tree build output, torchburn_b200/lib, built by
// `python -m torchburn_b200.build`, which needs nvcc); the CUDA runtime is linked into that
// library already, nothing else is required here.
use std::env;
use std::path::PathBuf;

fn main() {
    let dir = env::var("TORCHBURN_B200_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../torchburn_b200/lib")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=torchburn_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
    println!("cargo:rerun-if-env-changed=TORCHBURN_B200_LIB_DIR");
    println!("cargo:rerun-if-changed=../../include/torchburn_b200.h");
}
