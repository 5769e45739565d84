// Links libb2q.so (built by `python -m oxicuda_b200._build`).  B2Q_LIB_DIR names the directory that holds it;
// the library links the CUDA runtime statically, so nothing else is needed at link time.
use std::env;

fn main() {
    println!("cargo:rerun-if-env-changed=B2Q_LIB_DIR");
    if let Ok(dir) = env::var("B2Q_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=b2q");
    // device memory for the host-slice convenience paths of the wrapper crates
    println!("cargo:rustc-link-lib=dylib=cudart");
}
