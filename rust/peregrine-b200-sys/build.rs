// Links the shared library built by `python -m peregrine_b200.build`.  PEREGRINE_B200_LIB_DIR names the directory that
// holds libperegrine_b200.so (peregrine_b200/lib in this repository).
fn main() {
    if let Ok(dir) = std::env::var("PEREGRINE_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=peregrine_b200");
    println!("cargo:rerun-if-env-changed=PEREGRINE_B200_LIB_DIR");
}
