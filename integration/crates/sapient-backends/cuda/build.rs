//! Links libsapient_cuda.so. SAPIENT_CUDA_LIB_DIR names the directory that holds it (the `sapient_b200/` directory of
//! the CUDA backend's source tree after `python -m sapient_b200.build`, or wherever the .so was installed).
fn main() {
    println!("cargo:rerun-if-env-changed=SAPIENT_CUDA_LIB_DIR");
    let dir = std::env::var("SAPIENT_CUDA_LIB_DIR")
        .expect("set SAPIENT_CUDA_LIB_DIR to the directory that holds libsapient_cuda.so");
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=sapient_cuda");
    // the library is found at run time next to where it was linked from
    println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
}
