// Links libvolta_b200.so.  VOLTA_B200_LIB_DIR points at the directory that holds it
// (volta_b200/ in this repository after `python volta_b200/build.py`).
fn main() {
    if let Ok(dir) = std::env::var("VOLTA_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=volta_b200");
    println!("cargo:rerun-if-env-changed=VOLTA_B200_LIB_DIR");
}
