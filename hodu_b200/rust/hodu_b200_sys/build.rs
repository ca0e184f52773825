// Builds libhodu_b200.a from the CUDA sources with nvcc (sm_100a only) and tells cargo how to
// link it.  Stands where crates/hodu_cuda_kernels/build.rs:38-95 compiles the reference's
// kernels to PTX; here the objects carry their own host-side launch code, so the result is a
// static library with a C ABI instead of PTX strings.
//
// Environment: HODU_B200_SRC overrides the source directory (default: ../../csrc relative to
// this crate), CUDA_HOME the toolkit root (default /usr/local/cuda).
use std::{env, path::PathBuf, process::Command};

const SOURCES: &[&str] = &[
    "api", "gemm_tc", "gemm_simt", "gemm_f32", "gemm_f32_fused", "relayout", "splitk", "einsum", "conv", "conv_implicit", "cast", "host_pipeline",
];

fn main() {
    let out = PathBuf::from(env::var("OUT_DIR").expect("OUT_DIR"));
    let manifest = PathBuf::from(env::var("CARGO_MANIFEST_DIR").expect("CARGO_MANIFEST_DIR"));
    let src = env::var("HODU_B200_SRC").map(PathBuf::from).unwrap_or_else(|_| manifest.join("../../csrc"));
    let cuda = env::var("CUDA_HOME").unwrap_or_else(|_| "/usr/local/cuda".into());
    let nvcc = PathBuf::from(&cuda).join("bin/nvcc");
    let mut objs = Vec::new();
    for f in SOURCES {
        let obj = out.join(format!("{f}.o"));
        let status = Command::new(&nvcc)
            .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
                   "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-c"])
            .arg(src.join(format!("{f}.cu")))
            .arg("-o")
            .arg(&obj)
            .status()
            .expect("nvcc not found");
        assert!(status.success(), "nvcc failed on {f}.cu");
        objs.push(obj);
    }
    let lib = out.join("libhodu_b200.a");
    let status = Command::new("ar").arg("crs").arg(&lib).args(&objs).status().expect("ar not found");
    assert!(status.success(), "ar failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=static=hodu_b200");
    println!("cargo:rustc-link-search=native={cuda}/lib64");
    println!("cargo:rustc-link-lib=static=cudart_static");
    println!("cargo:rustc-link-lib=dylib=stdc++");
    println!("cargo:rustc-link-lib=dylib=dl");
    println!("cargo:rustc-link-lib=dylib=rt");
    println!("cargo:rustc-link-lib=dylib=pthread");
    println!("cargo:rerun-if-changed={}", src.display());
    println!("cargo:rerun-if-env-changed=HODU_B200_SRC");
    println!("cargo:rerun-if-env-changed=CUDA_HOME");
}
