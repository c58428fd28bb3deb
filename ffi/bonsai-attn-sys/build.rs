// UNBUILT (see Cargo.toml). Points the linker at libbonsai_attn.so: BONSAI_ATTN_LIB_DIR is the
// directory that holds it (bonsai_pot_b200/ of this repository after `python -c "import
// __graft_entry__ as g; g.build()"`, or wherever a packager installed it).
use std::env;

fn main() {
    println!("cargo:rerun-if-env-changed=BONSAI_ATTN_LIB_DIR");
    println!("cargo:rerun-if-changed=../../include/bonsai_attn.h");
    match env::var("BONSAI_ATTN_LIB_DIR") {
        Ok(dir) => {
            println!("cargo:rustc-link-search=native={dir}");
            println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
        }
        Err(_) => println!("cargo:warning=BONSAI_ATTN_LIB_DIR is not set: relying on the default library search path"),
    }
    println!("cargo:rustc-link-lib=dylib=bonsai_attn");
}
