// NOT COMPILED in this repository's build image (no Rust toolchain); see ../README.md.
//
// Links libhelium_b200.so.  The library is built by `python helium_b200/build.py` (nvcc, sm_100a) into
// helium_b200/lib/; HELIUM_B200_LIB_DIR overrides the directory.
use std::env;
use std::path::PathBuf;

fn main() {
    let dir = env::var("HELIUM_B200_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../helium_b200/lib")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=helium_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
    println!("cargo:rerun-if-env-changed=HELIUM_B200_LIB_DIR");
    println!("cargo:rerun-if-changed=../../include/helium_b200.h");
}
