{
  "targets": [{
    "target_name": "p0p_addon",
    "sources": ["addon.cc"],
    "include_dirs": ["../../include"],
    "libraries": ["-L<(module_root_dir)/..", "-lp0p", "-Wl,-rpath,<(module_root_dir)/.."],
    "cflags_cc": ["-std=c++17"]
  }]
}
