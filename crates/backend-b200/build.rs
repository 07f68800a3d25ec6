// Links against libeb200.so (built by `python -m harp_b200._build` in the backend's
// repository).  EB200_LIB_DIR names the directory that holds it.
fn main() {
    let dir = std::env::var("EB200_LIB_DIR").unwrap_or_else(|_| "/usr/local/lib".to_string());
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=eb200");
    println!("cargo:rerun-if-env-changed=EB200_LIB_DIR");
}
