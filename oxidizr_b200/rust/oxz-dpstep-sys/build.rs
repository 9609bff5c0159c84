// Links liboxz_dpstep.so. OXZ_DPSTEP_LIB_DIR names the directory that holds it (the `oxidizr_b200/` folder of the
// library's source tree after `python -m oxidizr_b200.build`); without it the system's default search path is used.
fn main() {
    println!("cargo:rerun-if-env-changed=OXZ_DPSTEP_LIB_DIR");
    if let Ok(dir) = std::env::var("OXZ_DPSTEP_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=oxz_dpstep");
}
