// NOT COMPILED in this repository's build image (no Rust toolchain); see Cargo.toml.
//
// Compiles the CUDA sources of libkhcuda_gqa for sm_100a with nvcc and links the crate against the result: the
// same single nvcc command `khalamari_b200/build.py` runs for the Python harness.
//
//   KHCUDA_GQA_CSRC   directory holding host_sdpa.cpp, sdpa_api.cu, sdpa_fp8.cu, kv_page_write.cu, bidi_block_sdpa.cu and their
//                     headers (default: ../khalamari_b200/csrc relative to this crate)
//   KHCUDA_GQA_DIR    use a prebuilt libkhcuda_gqa.so from this directory instead of compiling
//   NVCC              nvcc binary (default: nvcc on PATH, else /usr/local/cuda/bin/nvcc)
use std::env;
use std::path::{Path, PathBuf};
use std::process::Command;

const SOURCES: [&str; 6] =
    ["host_sdpa.cpp", "sdpa_api.cu", "sdpa_fp8.cu", "kv_page_write.cu", "bidi_block_sdpa.cu", "peer_exchange.cu"];
const HEADERS: [&str; 7] = ["common.h", "cuda_objects.h", "host_sdpa.h", "map_instance.h", "sdpa_map.cuh", "sdpa_tc.cuh", "sdpa_tm.cuh"];

fn main() {
    println!("cargo:rerun-if-env-changed=KHCUDA_GQA_DIR");
    println!("cargo:rerun-if-env-changed=KHCUDA_GQA_CSRC");
    println!("cargo:rerun-if-env-changed=NVCC");
    if let Ok(prebuilt) = env::var("KHCUDA_GQA_DIR") {
        link(Path::new(&prebuilt));
        return;
    }
    let manifest = PathBuf::from(env::var("CARGO_MANIFEST_DIR").expect("CARGO_MANIFEST_DIR"));
    let csrc = env::var("KHCUDA_GQA_CSRC").map(PathBuf::from).unwrap_or_else(|_| manifest.join("../khalamari_b200/csrc"));
    let out_dir = PathBuf::from(env::var("OUT_DIR").expect("OUT_DIR"));
    for name in SOURCES.iter().chain(HEADERS.iter()) {
        println!("cargo:rerun-if-changed={}", csrc.join(name).display());
    }
    println!("cargo:rerun-if-changed={}", csrc.join("../../include/kh_gqa.h").display());
    let nvcc = env::var("NVCC").unwrap_or_else(|_| {
        if Command::new("nvcc").arg("--version").output().is_ok() { "nvcc".into() } else { "/usr/local/cuda/bin/nvcc".into() }
    });
    let library = out_dir.join("libkhcuda_gqa.so");
    let mut command = Command::new(&nvcc);
    command
        .args(["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17"])
        .args(["-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-shared", "-t", "4", "-cudart", "static"]);
    if env::var("CARGO_FEATURE_MEASURE").is_ok() {
        command.arg("-DKH_GQA_MEASURE");
    }
    command.arg("-o").arg(&library);
    for name in SOURCES {
        command.arg(csrc.join(name));
    }
    let status = command.status().unwrap_or_else(|error| panic!("cannot run {nvcc}: {error}"));
    assert!(status.success(), "nvcc failed to build libkhcuda_gqa for sm_100a");
    link(&out_dir);
}

fn link(dir: &Path) {
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=khcuda_gqa");
    // the library links the CUDA runtime statically; the driver library comes with the GPU driver
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
}
