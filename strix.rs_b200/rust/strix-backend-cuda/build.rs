// Builds libstrix_cuda.so from the .cu / .cpp sources with nvcc for sm_100a only and links it.
// The same lines as strix.rs_b200/build.py (which is what the repository's own build runs).
use std::{env, path::PathBuf, process::Command};

fn main() {
    let root = PathBuf::from(env::var("STRIX_CUDA_SRC").unwrap_or_else(|_| "../..".into())); // the strix.rs_b200 directory
    let csrc = root.join("csrc");
    let include = root.join("../include");
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "/usr/local/cuda/bin/nvcc".into());
    let mut objs = Vec::new();
    for entry in std::fs::read_dir(&csrc).expect("csrc") {
        let p = entry.unwrap().path();
        let ext = p.extension().and_then(|e| e.to_str()).unwrap_or("");
        if ext != "cu" && ext != "cpp" { continue; }
        println!("cargo:rerun-if-changed={}", p.display());
        let obj = out.join(p.file_stem().unwrap()).with_extension("o");
        let ok = Command::new(&nvcc)
            .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
                   "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden"])
            .arg("-I").arg(&include).arg("-I").arg(&csrc)
            .arg("-c").arg(&p).arg("-o").arg(&obj)
            .status().expect("nvcc").success();
        assert!(ok, "nvcc failed on {}", p.display());
        objs.push(obj);
    }
    let lib = out.join("libstrix_cuda.so");
    let ok = Command::new(&nvcc).arg("-shared").arg("-o").arg(&lib).args(&objs)
        .args(["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart", "-ldl"])
        .status().expect("nvcc link").success();
    assert!(ok, "link failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=strix_cuda");
}
