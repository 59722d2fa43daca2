// Links the shared library built by `python datago_b200/build.py`.
// DATAGO_B200_LIB_DIR: the directory that holds libdatago_b200.so (the `datago_b200/` folder of this repository).
fn main() {
    println!("cargo:rerun-if-env-changed=DATAGO_B200_LIB_DIR");
    if let Ok(dir) = std::env::var("DATAGO_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=datago_b200");
}
