// ref_shim.cpp -- exposes the reference's own CPU oracle through a C ABI.
//
// TEST INFRASTRUCTURE ONLY.  The reference oracle (kvarn-evidence/oracle/bee_oracle.cpp in the
// reference repository) is a single-file command-line program whose functions are `static`.
// This translation unit compiles that file, unmodified and from where it lies (its path is
// given on the compiler command line as -DBEE_ORACLE_SRC="..."), and adds extern "C"
// wrappers around bee_quant_tile / bee_dequant_tile / f32_to_f16_rn so the parity tests can
// call the reference arithmetic directly.  No reference source is copied into this repository.
#define main bee_oracle_main
#include BEE_ORACLE_SRC
#undef main

extern "C" {

// bee_quant_tile (bee_oracle.cpp:318-357).  record must hold rows*cols*bits/8 + (2*rows+cols)*2 bytes.
int bee_ref_quant_tile(const float* tile, int rows, int cols, int bits, int iters, int cpu_order,
                       unsigned char* record, float* best_col, float* best_row, int* best_iter) {
    std::vector<uint8_t> rec;
    QuantMeta meta;
    bee_quant_tile(tile, rows, cols, bits, iters, rec, &meta, cpu_order != 0);
    std::memcpy(record, rec.data(), rec.size());
    if (best_col) std::memcpy(best_col, meta.best_col.data(), sizeof(float) * cols);
    if (best_row) std::memcpy(best_row, meta.best_row.data(), sizeof(float) * rows);
    if (best_iter) *best_iter = meta.best_iter;
    return (int)rec.size();
}

// bee_dequant_tile (bee_oracle.cpp:359-374)
void bee_ref_dequant_tile(const unsigned char* record, int rows, int cols, int bits, float* tile) {
    bee_dequant_tile(record, rows, cols, bits, tile);
}

// f32_to_f16_rn / f16_to_f32 (bee_oracle.cpp:49-100)
unsigned short bee_ref_f32_to_f16(float f) { return f32_to_f16_rn(f); }
float bee_ref_f16_to_f32(unsigned short h) { return f16_to_f32(h); }

// the program's own sub-commands (table, packtest, ...) for known-answer checks of its output
int bee_ref_main(int argc, char** argv) { return bee_oracle_main(argc, argv); }
}
