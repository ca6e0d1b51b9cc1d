// build.rs - compiles the hand-written sm_100a kernels into a static library and links it.
// Only active with `--features cuda`.  No fast-math, no flush-to-zero: the quantize kernel must
// reproduce IEEE f32 division and rounding bit for bit.
use std::{env, path::PathBuf, process::Command};

fn main() {
    if env::var_os("CARGO_FEATURE_CUDA").is_none() {
        return;
    }
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".into());
    let srcs = ["api.cu", "quantize.cu", "gemv.cu", "gemv_tma.cu", "prefill.cu", "shard.cu"];
    let mut objs = Vec::new();
    for s in srcs {
        let src = PathBuf::from("cuda").join(s);
        println!("cargo:rerun-if-changed={}", src.display());
        let obj = out.join(s).with_extension("o");
        let ok = Command::new(&nvcc)
            .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo"])
            .args(["-Xcompiler", "-fPIC,-fvisibility=hidden", "-Iinclude", "-c"])
            .arg(&src)
            .arg("-o")
            .arg(&obj)
            .status()
            .expect("nvcc not found")
            .success();
        assert!(ok, "nvcc failed on {}", src.display());
        objs.push(obj);
    }
    let lib = out.join("libnne_cuda.a");
    let ok = Command::new("ar").arg("rcs").arg(&lib).args(&objs).status().unwrap().success();
    assert!(ok, "ar failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=static=nne_cuda");
    let cuda = env::var("CUDA_HOME").unwrap_or_else(|_| "/usr/local/cuda".into());
    println!("cargo:rustc-link-search=native={cuda}/lib64");
    println!("cargo:rustc-link-lib=static=cudart_static");
    println!("cargo:rustc-link-lib=dylib=stdc++");
    println!("cargo:rustc-link-lib=dylib=dl");
    println!("cargo:rustc-link-lib=dylib=rt");
    println!("cargo:rustc-link-lib=dylib=pthread");
}
