// Compile-time target selection for the masked-attention group.
//
// The reference selects kernel families with a -DFA_TARGETS=<bits> mask
// (csrc/arch_targets.h:37-61: bit0 sm70, bit1 sm80-119, bit2 sm120).  This build
// adds one bit for data-centre Blackwell and ships only that family:
//
//   FA_TGT_SM100 (0x8)  compute capability 10.x, compiled for sm_100a
//
// A host runtime that also carries the reference's families would inject the bit
// for architectures 100-119 ahead of the sm8x rule and route `major == 10` to
// fa_mask_fwd_sm100().  Unlike the reference's process-wide cached gpu_major()
// (csrc/arch_targets.h:67-79), the launcher here caches per device ordinal.
#pragma once

#ifndef FA_TARGETS
#define FA_TARGETS 0x8
#endif

#define FA_TGT_SM70  0x1
#define FA_TGT_SM8X  0x2
#define FA_TGT_SM120 0x4
#define FA_TGT_SM100 0x8

#if FA_TARGETS & FA_TGT_SM100
#  define FA_HAS_SM100 1
#else
#  define FA_HAS_SM100 0
#endif

#if !FA_HAS_SM100
#  error "this library only contains the sm_100a kernels; build with FA_TARGETS including 0x8"
#endif
