// Links libb200attn.so. B200ATTN_LIB_DIR names the folder that holds it (the Makefile of
// candle-rocm-vulkan_b200/csrc writes it into candle-rocm-vulkan_b200/).
fn main() {
    println!("cargo:rerun-if-env-changed=B200ATTN_LIB_DIR");
    if let Ok(dir) = std::env::var("B200ATTN_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=b200attn");
}
