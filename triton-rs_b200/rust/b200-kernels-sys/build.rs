// Link against libb200_kernels.so; B200_KERNELS_LIB_DIR names the directory that holds it.
fn main() {
    if let Ok(dir) = std::env::var("B200_KERNELS_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rerun-if-env-changed=B200_KERNELS_LIB_DIR");
}
