// UNCOMPILED: written without a Rust toolchain at hand (see src/lib.rs).
//
// Compiles the CUDA sources of the library with nvcc for sm_100a and links them into the crate, the way
// krea2_hrx_b200/build.py builds libkrea2_b200.so.  Where the reference's build.rs embeds its Loom kernel
// sources for compilation at run time (build.rs:7-40), this one compiles ahead of time: the kernels are
// templates over the epilogue and the tile, not text specialised per sequence length.
use std::path::PathBuf;

const SOURCES: &[&str] = &[
    "api.cu", "prepare.cu", "gemm_i8.cu", "session.cu", "quantized.cu", "attention.cu", "sampler.cu", "checkpoint.cu",
];

fn main() {
    let root = PathBuf::from(std::env::var("CARGO_MANIFEST_DIR").unwrap()).join("..");
    let csrc = root.join("krea2_hrx_b200").join("csrc");
    let mut build = cc::Build::new();
    build
        .cuda(true)
        .cudart("shared")
        .flag("-gencode")
        .flag("arch=compute_100a,code=sm_100a")
        .flag("-lineinfo")
        .flag("-O3")
        .flag("-std=c++17")
        .flag("--expt-relaxed-constexpr")
        .include(root.join("include"));
    for source in SOURCES {
        let path = csrc.join(source);
        println!("cargo:rerun-if-changed={}", path.display());
        build.file(path);
    }
    println!("cargo:rerun-if-changed={}", csrc.join("common.cuh").display());
    println!("cargo:rerun-if-changed={}", root.join("include").join("krea2_b200.h").display());
    build.compile("krea2_b200");
    println!("cargo:rustc-link-lib=cudart");
    println!("cargo:rustc-link-lib=stdc++");
}
