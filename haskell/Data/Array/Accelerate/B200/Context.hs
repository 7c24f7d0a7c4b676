-- |
-- Module      : Data.Array.Accelerate.B200.Context
-- Description : Execution contexts: one per GPU (or per CUDA context handed in by the caller)
--
-- NOT COMPILED HERE: the build machine of this repository has no GHC.
--
-- Takes the place of Data/Array/Accelerate/CUDA/Context.hs:44-127 and the
-- default-context selection of CUDA/State.hs:111-132.  A context owns the
-- library's memory table, stream and event reservoirs and its share of the
-- kernel cache; all of that lives behind the C ABI.
--
module Data.Array.Accelerate.B200.Context (

  Context(..), create, fromCUcontext, destroy, defaultContext, withContext, performGCWith,

) where

import Control.Concurrent.MVar
import Control.Exception
import Foreign
import Foreign.C
import System.IO.Unsafe

import Data.Array.Accelerate.B200.FFI

-- | The library serialises calls on one context itself (a recursive mutex);
-- the MVar keeps one Haskell thread at a time inside a multi-call sequence
-- such as compile-then-run (the reference pushes and pops the CUDA context
-- around every evalCUDA, CUDA/State.hs:84-92).
data Context = Context
  { ctxHandle :: !(ForeignPtr AccbContext)
  , ctxDevice :: !Int
  , ctxLock   :: !(MVar ())
  }

instance Eq Context where
  a == b = ctxHandle a == ctxHandle b

-- | A context on the primary CUDA context of the given device.
create :: Int -> IO Context
create dev = fromCUcontext dev nullPtr

-- | A context that runs inside a CUDA context the caller owns
-- (accelerateCreate's second argument, include/AccFFI.h:21).
fromCUcontext :: Int -> Ptr () -> IO Context
fromCUcontext dev cu =
  alloca $ \out -> do
    st <- c_contextCreate (fromIntegral dev) cu out
    if st /= statusOK
      then do msg <- peekCString =<< c_lastError nullPtr
              throwIO (ErrorCall ("accelerate-b200: " ++ msg))
      else do h  <- peek out
              fp <- newForeignPtr_ h          -- released by 'destroy' (or at exit)
              Context fp dev <$> newMVar ()

destroy :: Context -> IO ()
destroy ctx = withForeignPtr (ctxHandle ctx) $ \h -> () <$ c_contextDestroy h

-- | Device 0, created on first use and shared by 'run' and 'run1'.
{-# NOINLINE defaultContext #-}
defaultContext :: Context
defaultContext = unsafePerformIO (create 0)

withContext :: Context -> (Ptr AccbContext -> IO a) -> IO a
withContext ctx k = withMVar (ctxLock ctx) $ \_ -> withForeignPtr (ctxHandle ctx) k

performGCWith :: Context -> IO ()
performGCWith ctx = withContext ctx $ \h -> throwOnError h =<< c_reclaim h
