// Points the linker at libratchet_cuda.so (built by `python -m ratchet_b200._build`).
fn main() {
    let dir = std::env::var("RATCHET_CUDA_LIB_DIR").unwrap_or_else(|_| {
        let manifest = std::env::var("CARGO_MANIFEST_DIR").unwrap();
        format!("{manifest}/../../ratchet_b200")
    });
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=ratchet_cuda");
    println!("cargo:rerun-if-env-changed=RATCHET_CUDA_LIB_DIR");
}
