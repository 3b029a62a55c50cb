// Keeps the host library non-empty until the packing / trajectory sources are built.
extern "C" __attribute__((visibility("default"))) int tb_host_abi_version() { return 1; }
