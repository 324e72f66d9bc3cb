// Links the shared library built by `python burn-mamba_b200/build.py` (nvcc, sm_100a).
// BM_B200_LIB_DIR = directory that holds libbm_b200.so.
fn main() {
    let dir = std::env::var("BM_B200_LIB_DIR").expect("set BM_B200_LIB_DIR to the directory of libbm_b200.so");
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=bm_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    println!("cargo:rerun-if-env-changed=BM_B200_LIB_DIR");
}
