// Tells cargo where libingot_cuda.so lives.  INGOT_CUDA_LIB_DIR = the directory that holds the library
// (the checkout's ingot_b200/ after `python -m ingot_b200.build`, or wherever it was installed).
fn main() {
    println!("cargo:rerun-if-env-changed=INGOT_CUDA_LIB_DIR");
    if let Ok(dir) = std::env::var("INGOT_CUDA_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=ingot_cuda");
}
