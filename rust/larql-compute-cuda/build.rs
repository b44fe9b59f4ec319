//! Locates (or builds) liblarql_b200.so and tells cargo to link it.
//!
//! The in-tree precedent for a natively built kernel is crates/larql-compute/build.rs:1-27 (cc-built C).
//! Here the library is built by the repository's own driver (`python -m larql_b200.build`, which runs
//! nvcc -gencode arch=compute_100a,code=sm_100a on every file under larql_b200/csrc), because the kernels
//! need nvcc rather than a C compiler.
//!
//!   LARQL_B200_ROOT   checkout of the larql_b200 repository (required)
//!   LARQL_B200_SKIP_BUILD=1   link a prebuilt larql_b200/liblarql_b200.so without rebuilding

use std::path::PathBuf;
use std::process::Command;

fn main() {
    println!("cargo:rerun-if-env-changed=LARQL_B200_ROOT");
    println!("cargo:rerun-if-env-changed=LARQL_B200_SKIP_BUILD");
    let root = PathBuf::from(
        std::env::var("LARQL_B200_ROOT").expect("set LARQL_B200_ROOT to the larql_b200 checkout"),
    );
    let lib_dir = root.join("larql_b200");
    if std::env::var("LARQL_B200_SKIP_BUILD").is_err() {
        let status = Command::new("python")
            .args(["-m", "larql_b200.build"])
            .current_dir(&root)
            .status()
            .expect("could not run python -m larql_b200.build");
        assert!(status.success(), "building liblarql_b200.so failed");
    }
    assert!(
        lib_dir.join("liblarql_b200.so").exists(),
        "liblarql_b200.so not found under {}",
        lib_dir.display()
    );
    println!("cargo:rerun-if-changed={}", root.join("include/larql_cuda.h").display());
    println!("cargo:rerun-if-changed={}", lib_dir.join("csrc").display());
    println!("cargo:rustc-link-search=native={}", lib_dir.display());
    println!("cargo:rustc-link-lib=dylib=larql_b200");
    // the library is loaded from where it was built; a deployment copies it next to the binary instead
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", lib_dir.display());
}
