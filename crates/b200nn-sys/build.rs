//! Builds libb200nn from the CUDA sources of this repository with nvcc for sm_100a and links it.
//!
//! Environment:
//!   NVCC            path of nvcc (default /usr/local/cuda/bin/nvcc)
//!   B200NN_LIB_DIR  with the `prebuilt` feature: directory that already holds libb200nn.so
//!
//! There is one target architecture (compute_100a / sm_100a) and no fallback: the kernels use
//! tcgen05, tensor memory and bulk async copies, which exist on no other architecture.
use std::env;
use std::path::{Path, PathBuf};
use std::process::Command;

fn main() {
    let manifest = PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap());
    let repo = manifest.parent().unwrap().parent().unwrap().to_path_buf();
    let csrc = repo.join("async-gpu_b200").join("csrc");
    let include = repo.join("include");
    println!("cargo:rerun-if-changed={}", include.join("b200nn.h").display());
    println!("cargo:rerun-if-env-changed=NVCC");
    println!("cargo:rerun-if-env-changed=B200NN_LIB_DIR");

    if env::var("CARGO_FEATURE_PREBUILT").is_ok() {
        let dir = env::var("B200NN_LIB_DIR").expect("feature `prebuilt` needs B200NN_LIB_DIR");
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-lib=dylib=b200nn");
        return;
    }

    let nvcc = env::var("NVCC").unwrap_or_else(|_| "/usr/local/cuda/bin/nvcc".to_string());
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let mut objects = Vec::new();
    let mut sources: Vec<PathBuf> = std::fs::read_dir(&csrc)
        .expect("async-gpu_b200/csrc is missing")
        .filter_map(|e| e.ok().map(|e| e.path()))
        .filter(|p| p.extension().map(|x| x == "cu").unwrap_or(false))
        .collect();
    sources.sort();
    for src in &sources {
        println!("cargo:rerun-if-changed={}", src.display());
        let obj = out.join(src.file_stem().unwrap()).with_extension("o");
        run(Command::new(&nvcc)
            .args(["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17"])
            .args(["-Xcompiler", "-fPIC,-fvisibility=hidden"])
            .arg("-I").arg(&include)
            .arg("-I").arg(&csrc)
            .arg("-c").arg(src)
            .arg("-o").arg(&obj));
        objects.push(obj);
    }
    for h in ["common.h", "model.h", "device_utils.cuh", "tc_ptx.cuh"] {
        println!("cargo:rerun-if-changed={}", csrc.join(h).display());
    }
    let lib = out.join("libb200nn.so");
    run(Command::new(&nvcc)
        .arg("-shared")
        .arg("-o").arg(&lib)
        .args(&objects)
        .args(["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]));
    link_dir(&out);
}

fn link_dir(dir: &Path) {
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=b200nn");
    // the CUDA runtime is linked statically into libb200nn.so; the driver library comes with the driver
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
}

fn run(cmd: &mut Command) {
    let status = cmd.status().unwrap_or_else(|e| panic!("cannot run {cmd:?}: {e}"));
    assert!(status.success(), "{cmd:?} failed");
}
