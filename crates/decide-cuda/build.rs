// Points the linker at libdecide_cuda.so, built in-tree by `python -m decide_b200.build`
// (nvcc -gencode arch=compute_100a,code=sm_100a). DECIDE_CUDA_LIB_DIR overrides the directory.
fn main() {
    let dir = std::env::var("DECIDE_CUDA_LIB_DIR").unwrap_or_else(|_| {
        let manifest = std::path::PathBuf::from(std::env::var("CARGO_MANIFEST_DIR").unwrap());
        manifest.join("../../decide_b200").display().to_string()
    });
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=decide_cuda");
    println!("cargo:rerun-if-env-changed=DECIDE_CUDA_LIB_DIR");
}
