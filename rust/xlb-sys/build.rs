// Points the linker at libxlb.so.  XLB_LIB_DIR names the directory that holds it (the repository
// builds it in xlog_b200/); the library itself is built with `make -C xlog_b200/csrc`.
use std::env;
use std::path::PathBuf;

fn main() {
    let dir = env::var("XLB_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../xlog_b200")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=xlb");
    println!("cargo:rerun-if-env-changed=XLB_LIB_DIR");
}
