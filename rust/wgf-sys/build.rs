// Points the linker at libwgf.so.  WGF_LIB_DIR is the directory that holds it (the package directory
// wgpu-kernal-fusion_b200/ after `python build.py`).
fn main() {
    println!("cargo:rerun-if-env-changed=WGF_LIB_DIR");
    if let Ok(dir) = std::env::var("WGF_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=wgf");
}
