// build.rs - compiles the hand-written sm_100a kernels into a static library and links it.
// Only active with `--features cuda`.  No fast-math, no flush-to-zero: the quantize kernel must
// reproduce IEEE f32 division and rounding bit for bit.
use std::{env, fs, path::PathBuf, process::Command};

fn main() {
    if env::var_os("CARGO_FEATURE_CUDA").is_none() {
        return;
    }
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".into());
    // Every kernel file under cuda/ (a copy of this backend's csrc/: *.cu, *.cuh) - a glob, not a
    // list, so a new kernel file is built without touching this script.
    println!("cargo:rerun-if-changed=cuda");
    println!("cargo:rerun-if-changed=include/nne_cuda.h");
    let mut srcs: Vec<PathBuf> = fs::read_dir("cuda")
        .expect("cuda/ directory with the kernel sources")
        .filter_map(|e| e.ok().map(|e| e.path()))
        .filter(|p| p.extension().map_or(false, |x| x == "cu"))
        .collect();
    srcs.sort();
    assert!(!srcs.is_empty(), "no .cu files under cuda/");
    let mut objs = Vec::new();
    for src in &srcs {
        println!("cargo:rerun-if-changed={}", src.display());
        let obj = out.join(src.file_name().unwrap()).with_extension("o");
        let ok = Command::new(&nvcc)
            .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo"])
            .args(["--fmad=true", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-c"])
            .arg(src)
            .arg("-o")
            .arg(&obj)
            .status()
            .expect("nvcc not found")
            .success();
        assert!(ok, "nvcc failed on {}", src.display());
        objs.push(obj);
    }
    let lib = out.join("libnne_cuda.a");
    let _ = fs::remove_file(&lib);
    let ok = Command::new("ar").arg("rcs").arg(&lib).args(&objs).status().unwrap().success();
    assert!(ok, "ar failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=static=nne_cuda");
    let cuda = env::var("CUDA_HOME").unwrap_or_else(|_| "/usr/local/cuda".into());
    println!("cargo:rustc-link-search=native={cuda}/lib64");
    println!("cargo:rustc-link-search=native={cuda}/lib64/stubs");
    println!("cargo:rustc-link-lib=static=cudart_static");
    println!("cargo:rustc-link-lib=dylib=cuda"); // cuTensorMapEncodeTiled is resolved through the driver
    println!("cargo:rustc-link-lib=dylib=stdc++");
    println!("cargo:rustc-link-lib=dylib=dl"); // NCCL is resolved at run time with dlopen, not linked
    println!("cargo:rustc-link-lib=dylib=rt");
    println!("cargo:rustc-link-lib=dylib=pthread");
}
