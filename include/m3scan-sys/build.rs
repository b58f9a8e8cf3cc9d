// Link against libm3scan.so; M3SCAN_LIB_DIR names the directory that holds it
// (mamba_trainer_b200/ after `python -m mamba_trainer_b200.build`).  Not compiled in this repository's image.
fn main() {
    if let Ok(dir) = std::env::var("M3SCAN_LIB_DIR") {
        println!("cargo:rustc-link-search=native={}", dir);
    }
    println!("cargo:rustc-link-lib=dylib=m3scan");
    println!("cargo:rerun-if-env-changed=M3SCAN_LIB_DIR");
}
