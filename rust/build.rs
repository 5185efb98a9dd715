//! Builds libflat_attention_b200 from the .cu sources for sm_100a with nvcc and links it.
//!
//! Environment: `NVCC` (default `nvcc`), `FLAT_ATTENTION_PREBUILT` = directory that already holds
//! `libflat_attention_b200.so` (skips the build).  With the `oracle-pin` feature the C++ restatement of the
//! scalar oracle (oracle/flat_oracle.cpp) is compiled with the host compiler and linked as well.
use std::env;
use std::path::{Path, PathBuf};
use std::process::Command;

fn run(cmd: &mut Command) {
    let status = cmd.status().unwrap_or_else(|e| panic!("cannot run {:?}: {e}", cmd));
    assert!(status.success(), "{:?} failed with {status}", cmd);
}

fn main() {
    let manifest = PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap());
    let root = manifest.parent().unwrap().to_path_buf();
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let csrc = root.join("flat-attention_b200").join("csrc");
    println!("cargo:rerun-if-changed={}", csrc.display());
    println!("cargo:rerun-if-changed={}", root.join("include").display());
    println!("cargo:rerun-if-env-changed=FLAT_ATTENTION_PREBUILT");

    let lib_dir = match env::var("FLAT_ATTENTION_PREBUILT") {
        Ok(dir) => PathBuf::from(dir),
        Err(_) => {
            let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".to_string());
            let mut objects = Vec::new();
            let mut sources: Vec<PathBuf> = std::fs::read_dir(&csrc)
                .expect("csrc directory")
                .filter_map(|e| e.ok().map(|e| e.path()))
                .filter(|p| p.extension().map(|x| x == "cu").unwrap_or(false))
                .collect();
            sources.sort();
            for src in &sources {
                let obj = out.join(Path::new(src.file_stem().unwrap()).with_extension("o"));
                run(Command::new(&nvcc)
                    .args(["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17"])
                    .args(["-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-c"])
                    .arg(src)
                    .arg("-o")
                    .arg(&obj));
                objects.push(obj);
            }
            let lib = out.join("libflat_attention_b200.so");
            run(Command::new(&nvcc)
                .args(["-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o"])
                .arg(&lib)
                .args(&objects)
                .arg("-ldl"));
            out.clone()
        }
    };
    println!("cargo:rustc-link-search=native={}", lib_dir.display());
    println!("cargo:rustc-link-lib=dylib=flat_attention_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", lib_dir.display());

    if env::var("CARGO_FEATURE_ORACLE_PIN").is_ok() {
        let cxx = env::var("CXX").unwrap_or_else(|_| "g++".to_string());
        let lib = out.join("libflat_oracle.so");
        // the flags of oracle/Makefile: no FMA contraction, no fast-math, glibc libm
        run(Command::new(&cxx)
            .args(["-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-pthread", "-o"])
            .arg(&lib)
            .arg(root.join("oracle").join("flat_oracle.cpp")));
        println!("cargo:rustc-link-search=native={}", out.display());
        println!("cargo:rustc-link-lib=dylib=flat_oracle");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{}", out.display());
    }
}
