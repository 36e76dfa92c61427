/* Empty stand-in for the THC/THC.h header that PyTorch removed: upstream's three .cu files
   include it (cuda/forward.cu:7, cuda/backward.cu:6, cuda/utils.cu:7) but use nothing from it. */
