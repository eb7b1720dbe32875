// build.rs for hanzo-quant with the B200 library: NOT COMPILED in this repository (no Rust toolchain in the
// build image).  Replaces the CUDA branch of hanzo-quant/build.rs:55-121.  The kernels are sm_100a only, so there is
// no compute-capability switch and no dummy sources: every optional-kernel cfg the crate tests for is set.
use std::{env, path::PathBuf, process::Command};

fn main() {
    println!("cargo:rerun-if-changed=build.rs");
    println!("cargo:rerun-if-env-changed=HQ_B200_SRC");
    println!("cargo:rerun-if-env-changed=CUDA_NVCC_FLAGS");

    // where engine_b200/csrc and include/ live (a checkout of this repository)
    let src = PathBuf::from(env::var("HQ_B200_SRC").expect("set HQ_B200_SRC to the hanzoquant_b200 checkout"));
    let csrc = src.join("engine_b200").join("csrc");
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".into());

    let mut objects = Vec::new();
    for entry in std::fs::read_dir(&csrc).expect("csrc directory") {
        let path = entry.unwrap().path();
        if path.extension().map(|e| e == "cu").unwrap_or(false) {
            println!("cargo:rerun-if-changed={}", path.display());
            let obj = out.join(path.file_stem().unwrap()).with_extension("o");
            let mut cmd = Command::new(&nvcc);
            cmd.args(["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17"])
                .args(["-Xcompiler", "-fPIC", "-c"])
                .arg(&path)
                .arg("-o")
                .arg(&obj);
            if let Ok(extra) = env::var("CUDA_NVCC_FLAGS") {
                cmd.args(["--compiler-options", &extra]);
            }
            assert!(cmd.status().expect("nvcc").success(), "nvcc failed on {}", path.display());
            objects.push(obj);
        }
    }
    // the reference links `hanzoquant` (build.rs:119): keep the name so nothing else changes
    let lib = out.join("libhanzoquant.a");
    let _ = std::fs::remove_file(&lib);
    assert!(Command::new("ar").arg("crs").arg(&lib).args(&objects).status().expect("ar").success());

    println!("cargo:rustc-link-search={}", out.display());
    println!("cargo:rustc-link-lib=hanzoquant");
    println!("cargo:rustc-link-lib=dylib=cudart");
    println!("cargo:rustc-link-lib=dylib=cuda"); // cuTensorMapEncodeTiled is resolved through the runtime, the
                                                 // driver library only has to be loadable
    println!("cargo:rustc-link-lib=dylib=stdc++");

    // optional-kernel switches of the crate (hanzo-quant/build.rs:82-93): all present
    for cfg in [
        "has_blockwise_fp8_kernels",
        "has_scalar_fp8_kernels",
        "has_vector_fp8_kernels",
        "has_mxfp4_kernels",
        "has_mxfp4_wmma_kernels",
        "has_b200_kernels",
    ] {
        println!("cargo:rustc-cfg={cfg}");
    }
}
